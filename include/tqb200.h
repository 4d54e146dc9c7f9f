/*
 * tqb200 — C ABI of the B200-native compressed-KV hot path (append/encode + decode-on-codes
 * attention) that sits behind TurboQuant Pro's TurboQuantKVCache.
 *
 * The reference has no C ABI on this path: its boundary is the Python class
 * TurboQuantKVCache (turboquant_pro/core.py:818-1307), the two stateless quantisers it
 * wires together (turboquant_pro/per_channel_kv.py:146-539 for keys,
 * turboquant_pro/core.py:139-654 for values) and the launch signature of its fused CuPy
 * kernel (turboquant_pro/kv_kernel.py:255-381).  Every entry point below names the
 * reference method(s) it replaces.
 *
 * Conventions
 *  - Plain C.  Every function returns an int32 status: TQ_OK (0) or a negative TQ_ERR_*.
 *    No exception crosses the boundary; tq_last_error() gives a message for the calling
 *    thread's most recent failure.
 *  - The library allocates NO device memory.  The caller asks tq_ctx_sizes() how many
 *    bytes each region needs, allocates them (cudaMalloc, a torch tensor, an arena ...)
 *    and hands the device pointers to tq_ctx_create().  The regions must stay alive until
 *    tq_ctx_destroy() and must be zero-filled before tq_ctx_create().
 *  - `stream` arguments are cudaStream_t passed as void*; NULL is the legacy default
 *    stream.  All device work of a call is enqueued on that stream and the call returns
 *    without synchronising unless it says otherwise.
 *  - A context is not thread-safe; use one per thread or serialise calls.  Contexts on
 *    different devices are independent.
 *  - One context holds n_layers x n_seqs independent two-tier caches (one reference
 *    TurboQuantKVCache each) that share geometry, rotation and codebooks.
 */
#ifndef TQB200_H
#define TQB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_VERSION 100

enum {
  TQ_OK = 0,
  TQ_ERR_INVALID = -1,      /* bad argument (shape, range, null pointer)            */
  TQ_ERR_UNSUPPORTED = -2,  /* geometry the kernels do not implement                 */
  TQ_ERR_CUDA = -3,         /* a CUDA runtime call failed; see tq_last_error()       */
  TQ_ERR_CAPACITY = -4,     /* append beyond max_tokens_per_seq or a full outlier pool */
  TQ_ERR_EMPTY = -5,        /* decode on a sequence with no tokens                   */
  TQ_ERR_NO_DEVICE = -6     /* no CUDA device / wrong architecture                   */
};

/* element type of incoming K/V tokens, of the hot window that stores them, and of q */
enum { TQ_F32 = 0, TQ_F16 = 1, TQ_BF16 = 2 };

/* Per-channel 4-bit key grids (per_channel_kv.py:285-401): dense value = mean + scale *
 * grid[code].  The three that kv_fused_pck.py:54-94 gives an affine form for:
 *   TQ_KEYS_NF4_ASYM  mean over the block's tokens, scale = max|x - mean|, NF4 grid (0 keeps
 *                     the value of the field that used to be reserved)
 *   TQ_KEYS_NF4       mean = 0, scale = max|x|, NF4 grid
 *   TQ_KEYS_UNIFORM   mean = min, scale = (max - min) / 15, grid = 0..15, round-half-even
 *   TQ_KEYS_POLAR     the legacy key format (per_channel_keys=False, core.py:1022-1033): keys go
 *                     through the value quantiser, TurboQuantKV.compress(kind="key")
 *                     (core.py:542-607: norm + rotated Lloyd-Max codes); decode is
 *                     _cold_partials (kv_fused.py:84-98).  key_bits must equal value_bits (the
 *                     reference's fused_decode requires it too, core.py:1191-1192) and
 *                     outlier_frac must be 0.  Served by the general-shape decode kernel. */
enum { TQ_KEYS_NF4_ASYM = 0, TQ_KEYS_NF4 = 1, TQ_KEYS_UNIFORM = 2, TQ_KEYS_POLAR = 3 };

/* Geometry of a context.  Fill the first block, then call tq_geom_finish(), which
 * validates it and derives the rest. */
typedef struct tq_geom {
  /* --- caller-provided --------------------------------------------------------- */
  int32_t n_layers;
  int32_t n_seqs;
  int32_t n_kv_heads;
  int32_t n_q_heads;          /* multiple of n_kv_heads; q head i reads KV head i / G  */
  int32_t head_dim;           /* 128                                                   */
  int32_t key_bits;           /* 4                                                     */
  int32_t value_bits;         /* 3 or 4                                                */
  int32_t hot_window;         /* tokens kept uncompressed, 2..512                      */
  int32_t kv_dtype;           /* TQ_F32 / TQ_F16 / TQ_BF16: tokens in, hot window      */
  int32_t max_tokens_per_seq;
  int32_t key_mode;           /* TQ_KEYS_*                                             */
  double outlier_frac;        /* per-channel fp16 outlier fraction, 0 disables         */
  /* --- derived by tq_geom_finish ------------------------------------------------ */
  int32_t group;              /* G = n_q_heads / n_kv_heads                            */
  int32_t block_tokens;       /* tokens per cold block = (hot_window + 1) / 2          */
  int32_t block_tokens_pad;   /* block_tokens rounded up to a multiple of 16           */
  int32_t hot_cap;            /* ring capacity: multiple of block_tokens > hot_window  */
  int32_t max_blocks;         /* cold blocks per sequence at max_tokens_per_seq        */
  int32_t outlier_k;          /* outliers kept per channel and block (before ties)     */
  int32_t k_bytes;            /* page section sizes in bytes ...                       */
  int32_t v_bytes;
  int32_t v_off, norm_off, scale_off, mean_off;
  int32_t page_bytes;         /* ... and the page stride (multiple of 128)             */
  int32_t pool_entries;       /* outlier-pool entries per (layer, seq, kv head)        */
  int32_t max_splits;         /* partial slots per (seq, kv head) in the scratch area  */
  int32_t hdr_off;            /* page header: outlier count, pool offset, row starts   */
  int32_t ent_off;            /* the page's own by-token copy of its outliers            */
  int32_t reserved_;
} tq_geom;

/* Byte sizes of the device regions a context needs. */
typedef struct tq_sizes {
  size_t pages;      /* cold pages                                   */
  size_t hot_k;      /* hot-window rings of keys                     */
  size_t hot_v;      /* hot-window rings of values                   */
  size_t pool_dec;   /* outlier entries read by decode (4 B each)    */
  size_t pool_val;   /* outlier fp16 values kept for export (2 B)    */
  size_t page_meta;  /* per-page outlier offset/count                */
  size_t state;      /* sequence lengths, pool cursors, status word  */
  size_t tables;     /* rotation matrices, codebooks                 */
  size_t scratch;    /* decode partials                              */
} tq_sizes;

/* Device pointers to the regions, each at least the size tq_ctx_sizes() reported and
 * 256-byte aligned. */
typedef struct tq_buffers {
  void* pages;
  void* hot_k;
  void* hot_v;
  void* pool_dec;
  void* pool_val;
  void* page_meta;
  void* state;
  void* tables;
  void* scratch;
} tq_buffers;

typedef struct tq_ctx tq_ctx;

/* Library version (TQ_VERSION). */
int32_t tq_version(void);

/* Message of the calling thread's most recent failing call ("" if none). */
const char* tq_last_error(void);

/* Validates the caller-provided half of `g` and fills the derived half.
 * Mirrors the constructor checks of TurboQuantKVCache.__init__ (core.py:886-969) and
 * PerChannelKV.__init__ (per_channel_kv.py:195-227) for the supported format. */
int32_t tq_geom_finish(tq_geom* g);

/* Bytes of every device region for geometry `g` (after tq_geom_finish). */
int32_t tq_ctx_sizes(const tq_geom* g, tq_sizes* out);

/* Creates a context over caller-allocated, zero-filled device regions and uploads the
 * tables.  `pi` is the D x D rotation (row-major, host, float32; value decode computes
 * y @ pi), `pi_t` its transpose (value encode computes x @ pi_t), `centroids` the
 * 2^value_bits direction codebook and `boundaries` its 2^value_bits - 1 bin edges —
 * what TurboQuantKV.__init__ builds (core.py:229-260).  Synchronises `stream`. */
int32_t tq_ctx_create(const tq_geom* g, const tq_buffers* bufs, int32_t device,
                      const float* pi, const float* pi_t, const float* centroids,
                      const float* boundaries, void* stream, tq_ctx** out);

int32_t tq_ctx_destroy(tq_ctx* ctx);

/* Appends `n_tokens` tokens to each of the sequences [seq_begin, seq_begin + seq_count)
 * of `layer`, performing exactly the flushes the reference would perform had the tokens
 * been appended one at a time: TurboQuantKVCache.append + _flush_to_cold
 * (core.py:986-1038), i.e. PerChannelKV.compress (per_channel_kv.py:285-401) for keys
 * and TurboQuantKV.compress(kind="value") (core.py:542-607) for values.
 * `k`/`v` are device pointers of element type geom.kv_dtype; element (seq i, token t,
 * head h, channel d) is at  base + (i - seq_begin)*seq_stride + t*tok_stride +
 * h*head_stride + d  (strides in elements). */
int32_t tq_append(tq_ctx* ctx, int32_t layer, int32_t seq_begin, int32_t seq_count,
                  const void* k, const void* v, int32_t n_tokens, int64_t seq_stride,
                  int64_t tok_stride, int64_t head_stride, void* stream);

/* One decode step of attention for every sequence of `layer`, computed on the codes:
 * TurboQuantKVCache.fused_decode (core.py:1168-1265), whose result equals
 * get_keys/get_values + softmax(qK^T/sqrt(D))V.  `q` is [n_seqs][n_q_heads][D] of
 * `q_dtype`; `out` is [n_seqs][n_q_heads][D] float32.  Sequences with no tokens get
 * zeros.  Uses the context's scratch region, so two decodes of one context must not
 * overlap on the device. */
int32_t tq_decode(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype, float* out,
                  void* stream);

/* Sequence-split form of tq_decode for one long sequence spread over several devices:
 * attends only cold blocks [block_begin, block_end) and, if `with_hot` is non-zero, the
 * hot window, and writes the un-normalised state (m, l, o[D]) per query head to
 * `mlo` ([n_seqs][n_q_heads][2 + D] float32) instead of the final output.  The states
 * of all ranks, gathered rank-major, go to tq_lse_combine.  Generalises the per-page
 * partials of PreparedPCKBlock.partials (kv_fused_pck.py:211-236). */
int32_t tq_decode_partial(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype,
                          int32_t block_begin, int32_t block_end, int32_t with_hot, float* mlo,
                          void* stream);

/* Log-sum-exp merge of `n_parts` gathered states: merge_partials (kv_fused.py:139-153).
 * `mlo` is [n_parts][n_rows][2 + D] float32 (device), `out` [n_rows][D] float32. */
int32_t tq_lse_combine(const float* mlo, int32_t n_parts, int32_t n_rows, int32_t head_dim,
                       float* out, void* stream);

/* ---- exchange of the sequence-split states over peer memory ------------------------------
 * The reference merges the per-page partials of one device (merge_partials,
 * kv_fused.py:139-153) and leaves any exchange between devices to its caller.  A tq_xchg
 * replaces "all-gather the (m, l, o) states of every rank, then tq_lse_combine" by ONE kernel
 * per call: each rank stores its rows straight into every rank's region with peer stores
 * over NVLink, signals per row group, waits (bounded) for the same row group of the other
 * ranks and merges in rank order - bit-identical to tq_lse_combine on the gathered states.
 *
 * Life cycle, one object per rank: tq_xchg_create (allocates this rank's region with
 * cudaMalloc, zeroed) -> publish tq_xchg_ipc_handle to the other processes (64 bytes, any
 * transport) -> tq_xchg_open_peer for each of them (or tq_xchg_set_peer with the address
 * from tq_xchg_base when the ranks are GPUs of one process with peer access enabled) -> a
 * barrier of the caller's (every region must be zeroed before the first exchange) ->
 * tq_xchg_gather_merge any number of times, the same number on every rank ->
 * a barrier -> tq_xchg_destroy.  `rows` = n_seqs * n_q_heads; at most 16 ranks. */
typedef struct tq_xchg tq_xchg;
int32_t tq_xchg_create(int32_t device, int32_t rank, int32_t world, int32_t rows, int32_t head_dim,
                       tq_xchg** out);
int32_t tq_xchg_destroy(tq_xchg* x);
/* Size and device address of this rank's region. */
int64_t tq_xchg_region_bytes(const tq_xchg* x);
void* tq_xchg_base(const tq_xchg* x);
/* The CUDA IPC handle of this rank's region (`handle64`: 64 bytes of HOST memory). */
int32_t tq_xchg_ipc_handle(tq_xchg* x, void* handle64);
/* Maps the region of `peer_rank` (another process) from its IPC handle. */
int32_t tq_xchg_open_peer(tq_xchg* x, int32_t peer_rank, const void* handle64);
/* Uses `region` (device address valid in this process, e.g. tq_xchg_base of an object on
 * another GPU of the same process) as the region of `peer_rank`. */
int32_t tq_xchg_set_peer(tq_xchg* x, int32_t peer_rank, void* region);
/* One exchange.  `mlo`: this rank's states [rows][2 + D] float32 (tq_decode_partial's
 * output); `out`: [rows][D] float32.  `phases`: 3 = publish, wait and merge (the normal
 * call); 1 = publish only and 2 = wait and merge only, for callers that drive several ranks
 * from one stream and must not make a kernel wait for one that has not been launched yet.
 * If a peer's rows do not arrive within the wait limit, bit 0 of tq_xchg_status is set and
 * the affected rows of `out` are zero; the call itself still returns TQ_OK. */
int32_t tq_xchg_gather_merge(tq_xchg* x, const float* mlo, float* out, int32_t phases,
                             void* stream);
/* tq_decode_partial and tq_xchg_gather_merge in one call, with one kernel less on the critical
 * path: the kernel that merges the rank's own partials publishes its rows to the other ranks
 * and merges theirs itself.  `out` is the final [n_seqs][n_q_heads][D] float32 output, the
 * same bits as the two-call form.  `phases`: 3 (the normal call) or 1 (publish only; follow
 * with tq_xchg_gather_merge(..., phases = 2), see there).  Returns TQ_ERR_UNSUPPORTED where the
 * layer is not served by one launch of the tensor-core kernel or `xchg` was created for another
 * row count; the two-call form works everywhere. */
int32_t tq_decode_exchange(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype,
                           int32_t block_begin, int32_t block_end, int32_t with_hot, tq_xchg* xchg,
                           float* out, int32_t phases, void* stream);
/* Probes a wait makes before it gives up (each takes 0.1 us or more); 0 restores the default
 * (about half a second). */
int32_t tq_xchg_set_wait_limit(tq_xchg* x, int32_t probes);
/* Status word of this rank's exchanges (bit 0: a wait ran out).  Synchronises `stream`. */
int32_t tq_xchg_status(tq_xchg* x, int32_t* status, void* stream);

/* Dequantised keys and values of tokens [start, end) of one sequence, float32
 * [n_kv_heads][end - start][D] each (device pointers, either may be NULL):
 * TurboQuantKVCache.get_keys / get_values (core.py:1040-1117), bit-identical to
 * PerChannelKV.decompress (per_channel_kv.py:497-539) and TurboQuantKV.decompress
 * (core.py:619-654). */
int32_t tq_dequant_range(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t start, int32_t end,
                         float* k_out, float* v_out, void* stream);

/* Copies cold block `block` of (layer, seq) to HOST arrays in the reference's container
 * layout (CompressedPerChannelKV, per_channel_kv.py:103-143; CompressedKV,
 * core.py:96-136) for all KV heads: key_indices [H*S*D/2] (bit-reversed nibbles of
 * _pack_indices, per_channel_kv.py:87-93), nf4_scale/nf4_mean [H*D], outlier_idx
 * (ascending flat index into (H,S,D)) and outlier_val (fp16 bits) with capacity
 * `outlier_cap` (count returned in *n_outliers), value_indices (_pack_bits_cpu layout,
 * core.py:350-398) and value_norms [H*S].  With TQ_KEYS_POLAR the key container is a
 * CompressedKV too: key_indices receives the key codes packed like value_indices
 * (H*S*D*key_bits/8 bytes), nf4_scale the key norms [H*S] (give it that much room), nf4_mean
 * is left alone and there are no outliers.  Synchronises `stream`. */
int32_t tq_export_block(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t block,
                        uint8_t* key_indices, float* nf4_scale, float* nf4_mean,
                        int32_t* outlier_idx, uint16_t* outlier_val, int32_t outlier_cap,
                        int32_t* n_outliers, uint8_t* value_indices, float* value_norms,
                        void* stream);

/* The inverse of tq_export_block: writes cold block `block` of (layer, seq) from HOST arrays in
 * the reference's container layout (same arrays and orders as tq_export_block; key_mean is
 * the full [H*D] zero-point, zeros for symmetric NF4), i.e. what the reference's connector
 * reads back from a stored block (connectors/vllm_v1.py:150-196) without going through dense
 * tensors.  The cache of (layer, seq) must be cleared (length 0); blocks may be imported in
 * any order; tq_restore_hot then sets the length.  TQ_ERR_CAPACITY when the block or its
 * outliers do not fit.  Synchronises `stream`. */
int32_t tq_import_block(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t block,
                        const uint8_t* key_indices, const float* key_scale, const float* key_mean,
                        const int32_t* outlier_idx, const uint16_t* outlier_val,
                        int32_t n_outliers, const uint8_t* value_indices,
                        const float* value_norms, void* stream);

/* Completes a restore: (layer, seq) holds `n_tokens` tokens, of which the cold blocks were
 * imported with tq_import_block and the newest n_tokens - 256 * n_cold_blocks are given here
 * as DEVICE arrays hot_k / hot_v [tokens][n_kv_heads][128] of the context's K/V dtype, with
 * element strides tok_stride / head_stride (the hot window of TurboQuantKVCache,
 * core.py:986-1030, which the reference keeps uncompressed). */
int32_t tq_restore_hot(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t n_tokens,
                       const void* hot_k, const void* hot_v, int64_t tok_stride,
                       int64_t head_stride, void* stream);

/* Tokens currently held by (layer, seq): total, in cold blocks, in the hot window
 * (TurboQuantKVCache.length / cold_length / hot_length, core.py:971-984). */
int32_t tq_seq_lengths(const tq_ctx* ctx, int32_t layer, int32_t seq, int32_t* total,
                       int32_t* cold, int32_t* hot);

/* Bytes held by (layer, seq) counted like the reference's containers
 * (TurboQuantKVCache.memory_stats, core.py:1267-1296); needs the outlier counts, so it
 * synchronises `stream`. */
int32_t tq_memory_stats(tq_ctx* ctx, int32_t layer, int32_t seq, double* cold_bytes,
                        double* hot_bytes, void* stream);

/* Empties (layer, seq) — TurboQuantKVCache.clear (core.py:1298-1307); seq = -1 clears
 * every sequence of the layer. */
int32_t tq_clear(tq_ctx* ctx, int32_t layer, int32_t seq, void* stream);

/* Reads and clears the device status word.  Synchronises `stream`.
 *   bit 0 (1): an outlier pool overflowed and a block kept a truncated side-list;
 *   bit 1 (2): a bounded wait inside the tensor-core decode kernel ran out (a tile copy did
 *              not arrive within the limit), or one inside the tcgen05 value encoder.  The kernel then stops waiting and returns, so
 *              the device stays usable, but the `out` / `mlo` of that call is undefined:
 *              tq_decode itself has already returned TQ_OK (it does not synchronise), so a
 *              caller that wants the guarantee reads the status after the call. */
int32_t tq_status(tq_ctx* ctx, int32_t* flags, void* stream);

/* Chooses, for the whole process, the kernel that rotates and quantises values (and, in
 * TQ_KEYS_POLAR mode, keys) on tq_append — both implement PolarQuant.encode (core.py) and
 * write identical pages:
 *   1  (default) the rotation on tcgen05.mma with the accumulators in tensor memory, one CTA
 *      per SM.  Its waits for the products are bounded; if one runs out, bit 1 of the status
 *      word is set.
 *   0  the rotation on warp-level mma.sync instructions;
 *  -1  back to the default.
 * Not part of the reference's interface: a switch for measurements and tests. */
int32_t tq_set_value_encoder(int32_t kind);

/* Algorithmic bytes one tq_decode of `layer` reads (reference container sizes of every
 * cold block + the hot windows + q at the element size of the most recent decode's q_dtype,
 * float32 before the first one, + the float32 out), for roofline accounting. */
int32_t tq_decode_bytes(const tq_ctx* ctx, int32_t layer, double* bytes);

/* Number of kernels the most recent tq_decode / tq_append of this context launched. */
int32_t tq_last_launches(const tq_ctx* ctx);

/* tq_decode for callers that have no working memory to lend and may not allocate any (an
 * engine plugin that only receives q and out, a process whose device allocations are frozen
 * while it serves, a sandboxed extension).  It has no counterpart in the reference.  The
 * split-K partials go to a fixed 4.1 MiB array inside the library image instead of the
 * context's scratch region; nothing is allocated or freed.  Limit: n_seqs * n_q_heads <=
 * 1024, otherwise TQ_ERR_CAPACITY.  The array is shared by all contexts and streams of the
 * process on that GPU, so calls must not overlap on the device.  The first call on a device
 * resolves the array's device address; make it before any stream capture, and do not let two
 * threads make their first call on the same device at the same time (later calls only read
 * the remembered address).  Always runs the general-shape kernel; same result as tq_decode
 * within rounding. */
int32_t tq_decode_static_scratch(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype,
                                 float* out, void* stream);

/* The "sparse" zero-point of asymmetric NF4 keys (per_channel_kv.py:337-342, :517-522): the
 * per-channel mean is kept only on the channels whose mask byte is non-zero (the reference
 * derives the mask from the rotary wavelengths, dc_channel_mask at :233-241; the caller
 * computes it) and is 0 elsewhere.  `mask` is head_dim bytes of host memory; a null mask
 * restores the default (every channel).  Set it before the first append; blocks already
 * encoded keep the zero-points they were encoded with.  TQ_KEYS_NF4_ASYM only. */
int32_t tq_set_key_mean_mask(tq_ctx* ctx, const uint8_t* mask, void* stream);

/* The "bias" zero-point of asymmetric NF4 keys (per_channel_kv.py:327-336, :506-516): the
 * zero-point of a block is not measured but given — the reference derives it from the
 * model's key-projection bias rotated and averaged over the block's positions
 * (rope_averaged_bias at :243-267), so it depends only on the KV head and on where the block
 * starts.  `means` is host memory [max_blocks][n_kv_heads][head_dim] float32, entry b for the
 * block that starts at token b * block_tokens; it is copied into the tables region.  A null
 * pointer goes back to measured means.  Set it before the first append.  TQ_KEYS_NF4_ASYM
 * only; the byte accounting then counts no stored mean, like the reference. */
int32_t tq_set_key_bias_means(tq_ctx* ctx, const float* means, void* stream);

/* Selects the decode kernel: 0 = automatic (the tensor-core kernel where the geometry
 * allows: 256-token blocks, GQA group 1/2/4/8, any number of sequences; else the
 * general-shape kernel), 1 = always the general-shape float32 kernel.  Both compute the same
 * function; tests compare them; tq_last_kernel tells which one ran.  No counterpart in the
 * reference. */
int32_t tq_set_kernel(tq_ctx* ctx, int32_t which);

/* Which kernel the most recent tq_decode / tq_decode_partial / tq_decode_static_scratch of
 * this context ran: 0 none yet, 1 the tensor-core kernel, 2 the general-shape kernel.  The
 * reference likewise lets callers see which path served a call (it dispatches by capability,
 * kv_fused_pck.py:216-236); no direct counterpart. */
int32_t tq_last_kernel(const tq_ctx* ctx);

/* Test hook for the bounded waits of the tensor-core decode kernel (no counterpart in the
 * reference).  `wait_limit` > 0 replaces the number of probes a wait makes before it gives up
 * (0 restores the default, about half a second); `withhold_tile` >= 0 makes the first CTA of
 * later decodes never start the copy of that tile of its share, so that the wait for it runs
 * out and bit 1 of the status word is set (-1 switches this off).  Nothing faults and nothing
 * spins without bound; used by the tests of the error path. */
int32_t tq_debug_wait(tq_ctx* ctx, int32_t wait_limit, int32_t withhold_tile);

/* Pipeline trace of the tensor-core decode kernel (debugging aid, no counterpart in the
 * reference).  `on` switches stamping on or off for later tq_decode calls; if `stamps` is
 * non-null the 512 SM-clock stamps of the most recent traced decode (first CTA, 64 tiles x
 * 8 phases: copy wait/issue, prepare wait/start/done, consumer wait/start/done) are copied
 * to that HOST array.  Synchronises `stream`. */
int32_t tq_debug_trace(tq_ctx* ctx, int32_t on, uint64_t* stamps, void* stream);

/* Per-kernel timing for benchmarks (no counterpart in the reference, whose harnesses time
 * whole calls with time.perf_counter, benchmarks/p5_triton_bench.py:72-82).  While enabled,
 * tq_decode brackets its attention kernel and its combine kernel with CUDA events on the
 * launch stream (up to 4096 calls between reads). */
int32_t tq_profile_enable(tq_ctx* ctx, int32_t on);

/* Synchronises the recorded events and returns the summed attention-kernel and
 * combine-kernel milliseconds and the number of tq_decode calls they cover; resets. */
int32_t tq_profile_read(tq_ctx* ctx, double* attn_ms, double* combine_ms, int32_t* n_calls);

#ifdef __cplusplus
}
#endif
#endif /* TQB200_H */
