// Shared declarations of the tqb200 CUDA library: context object, device-memory layout
// helpers, element-type loaders.  Everything here is internal; the public surface is
// include/tqb200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "tqb200.h"

#define TQ_HD __host__ __device__ __forceinline__
#define TQ_DEV __device__ __forceinline__

constexpr int TQ_D = 128;          // head dimension the kernels are written for
constexpr int TQ_GROUP_TOK = 16;   // tokens per value-code group (one MMA k-step)
constexpr int TQ_MAX_K_OUT = 32;   // most outliers per channel the key encoder tracks
constexpr int TQ_MAX_G = 16;       // largest GQA group
constexpr int TQ_PART_STRIDE = 2 + TQ_D;  // floats per partial state (m, l, acc[D])

// Tail of a page, offsets from hdr_off: header | wide-channel codes | outliers by token
constexpr int TQ_WIDE = 4;          // channels per page whose codes are kept a second time
constexpr int TQ_SIDE_OFF = 64;     // uint16 x 256: the codes of the wide channels, per token
constexpr int TQ_ELL_SLOTS = 4;     // outliers of a token kept in its fixed slots
constexpr int TQ_ELL_OFF = TQ_SIDE_OFF + 512;            // fp16 delta [slots][256], then
constexpr int TQ_ELL_COL_OFF = TQ_ELL_OFF + TQ_ELL_SLOTS * 512;  // uint8 channel [slots][256]
constexpr int TQ_OVF_OFF = TQ_ELL_COL_OFF + TQ_ELL_SLOTS * 256;  // uint32 entries beyond the slots
constexpr int TQ_OVF_CAP = 112;
constexpr int TQ_TAIL_BYTES = TQ_OVF_OFF + TQ_OVF_CAP * 4;  // 4096
constexpr int TQ_PAGE_SPILLED = 1;  // header flag: use the pool's list, not the in-page copy

// device status word: bit 0, an outlier pool overflowed; bit 1, a bounded wait of the
// tensor-core decode kernel ran out (the call's output is then undefined)
constexpr int TQ_STATUS_POOL_OVERFLOW = 1;
constexpr int TQ_STATUS_WAIT_TIMEOUT = 2;

// which decode kernel served the most recent call (tq_last_kernel)
constexpr int TQ_KERNEL_NONE = 0, TQ_KERNEL_TENSOR_CORE = 1, TQ_KERNEL_GENERAL = 2;

// head of the scratch region as the tensor-core path uses it: trace stamps, then per launch a
// plan block followed by that launch's partials
constexpr size_t TQ_MMA_TRACE_BYTES = 4096;
constexpr size_t TQ_MMA_PLAN_BYTES = 8192;

// ---------------------------------------------------------------------------------------
// Device memory layout
//
// pages     [L][B][H][max_blocks] x page_bytes.  One page = one cold block of one KV head:
//             +0          key codes, token-major rows of 64 bytes, byte j of a row holds
//                         channel 2j in its low nibble and channel 2j+1 in its high nibble
//             +v_off      value codes in groups of 16 tokens (see v_field_* below)
//             +norm_off   value norms, float32 per token
//             +scale_off  key scale per channel (max |x - mean|), float32
//             +mean_off   key zero-point per channel, float32
//             +hdr_off    PageHeader (below), then at +TQ_SIDE_OFF one uint16 per token
//                         holding the codes of the TQ_WIDE widest channels (nibble i = code
//                         of wide channel i)
//             +ent_off    the page's own copy of its outliers, by token: the first
//                         TQ_ELL_SLOTS of every token as fp16 delta [slot][token] and uint8
//                         channel [slot][token] (empty slots are zero), then up to
//                         TQ_OVF_CAP further entries in pool format, ordered by token
// hot_k/v   [L][B][H][hot_cap][D] of kv_dtype; token at position p lives in slot p % hot_cap
// pool_dec  [L][B][H][pool_entries] uint32: fp16 delta | channel << 16 | token << 24
// pool_val  same shape, uint16: the outlier's fp16 value (kept for export / dequant)
// page_meta [L][B][H][max_blocks] {offset into the (l,b,h) pool slab, entry count}
// state     int32 seq_len[L][B]; uint32 pool_cursor[L][B][H]; int32 status[16]
// tables    float pi[D*D], pi_t[D*D], centroids[16], boundaries[16], nf4[16]
// scratch   decode partials
// ---------------------------------------------------------------------------------------

// First bytes of a page's tail.  The decode kernel reads the outliers from the page unless
// TQ_PAGE_SPILLED is set (more overflow entries than fit, or the pool slab was full).
struct PageHeader {
  uint32_t off, cnt;       // the page's PageMeta
  uint8_t wide[TQ_WIDE];   // channels with the largest scale, widest first
  uint16_t ovf_n, flags;   // overflow entries stored in the page; TQ_PAGE_* bits
  uint16_t ovf_start[5];   // first overflow entry of each 64-token strip, and the end
  uint16_t pad_[19];
};
static_assert(sizeof(PageHeader) == TQ_SIDE_OFF, "page header size");

// Row of channel d in the decode kernel's [channel][query row] copy of the query.  The
// fragment build reads channels 32c + 4j + i for c = 0..3 at once; the XOR spreads those
// four rows over different banks.  The in-page outlier slots store channels in this form.
TQ_HD int q_row(int d) { return d ^ ((d >> 5) << 1); }

struct PageMeta {
  uint32_t off;
  uint32_t cnt;
};

struct Tables {
  float pi[TQ_D * TQ_D];
  float pi_t[TQ_D * TQ_D];
  float centroids[16];
  float boundaries[16];
  float grid[16];  // key levels: NF4, or 0..15 for uniform keys
  uint8_t mean_mask[TQ_D];  // asymmetric NF4: channels that keep their mean (default all)
};

struct tq_ctx {
  tq_geom g;
  tq_buffers b;
  int device;
  // host mirror of the per-(layer, seq) token counts; the device copy in `state` is the
  // one kernels read, both are advanced together by tq_append
  std::vector<int32_t> len;
  int last_launches;
  int last_kernel = TQ_KERNEL_NONE;
  int last_q_dtype = TQ_F32;   // query element type of the most recent decode (byte accounting)
  bool force_generic = false;  // route every decode through the general-shape kernel
  bool trace_on = false;       // the tensor-core decode kernel stamps its pipeline phases
  int wait_limit = 0;          // probes per bounded wait of the decode kernel; 0 = default
  int withhold_tile = -1;      // test hook: the copy of this tile of CTA 0 is never started
  // optional per-kernel timing: event triples (before attention, after it, after combine)
  bool prof_on = false;
  int prof_n = 0;
  std::vector<cudaEvent_t> prof_ev;
  float h_centroids[16];
  float h_boundaries[16];
  // tensor maps (opaque 128-byte driver objects) of the two hot rings as 2-D arrays
  // [ring rows][128] of 16-bit elements, for the decode kernel's swizzled tile copies;
  // state 0: not built yet, 1: ready, -1: not available (float32 rings, or no driver entry)
  int mean_channels = TQ_D;  // channels with a stored mean, for the byte accounting
  bool bias_means = false;   // key zero-points come from the table behind the Tables struct
  alignas(64) unsigned char tmap_hot[2][128];
  int tmap_state = 0;
};

TQ_HD size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

TQ_HD int n_cold_blocks(int n_tokens, int hot_window, int block_tokens) {
  return n_tokens <= hot_window ? 0 : 1 + (n_tokens - hot_window - 1) / block_tokens;
}

TQ_HD size_t unit_index(const tq_geom& g, int layer, int seq, int head) {
  return ((size_t)layer * g.n_seqs + seq) * g.n_kv_heads + head;
}

TQ_HD size_t page_offset(const tq_geom& g, int layer, int seq, int head, int blk) {
  return (unit_index(g, layer, seq, head) * g.max_blocks + blk) * (size_t)g.page_bytes;
}

TQ_HD size_t hot_offset_elems(const tq_geom& g, int layer, int seq, int head) {
  return unit_index(g, layer, seq, head) * (size_t)g.hot_cap * TQ_D;
}

// state region
TQ_HD size_t state_len_off(const tq_geom&) { return 0; }
TQ_HD size_t state_cursor_off(const tq_geom& g) {
  return align_up((size_t)g.n_layers * g.n_seqs * 4, 256);
}
TQ_HD size_t state_status_off(const tq_geom& g) {
  return state_cursor_off(g) + align_up((size_t)g.n_layers * g.n_seqs * g.n_kv_heads * 4, 256);
}
TQ_HD size_t state_bytes(const tq_geom& g) { return state_status_off(g) + 256; }

// Value codes of a 16-token group.  Element (token t of the group, channel d) belongs to
// "lane" l = (d % 8) * 4 + (t % 8) / 2 and, inside that lane's record, to pair
// p = 2 * (d / 8) + t / 8; the pair packs tokens (t & ~1, t | 1) of channel d, the even
// token in the low bits.  A lane record is 32 pairs: 32 bytes at 4 bits, 24 bytes at 3
// bits.  Records are stored part-major ([part][lane]) in parts of 16 (4-bit) or 8 (3-bit)
// bytes, so that one warp reads a part with one conflict-free vector load, and the pair
// layout is exactly the A fragment of an m16n8k16 tensor-core tile whose rows are channels
// and whose k index is the token: lane (r, c) of a warp owns channels r, r+8, r+16, ...
// and tokens 2c, 2c+1, 2c+8, 2c+9.
TQ_HD int v_group_bytes(int bits) { return TQ_GROUP_TOK * TQ_D * bits / 8; }
TQ_HD int v_lane(int t, int d) { return (d & 7) * 4 + ((t & 7) >> 1); }
TQ_HD int v_pair(int t, int d) { return 2 * (d >> 3) + (t >> 3); }

// byte offset inside the group of byte `byte_in_record` of lane `l`'s record
TQ_HD int v_record_byte_off(int bits, int l, int byte_in_record) {
  if (bits == 4) return (byte_in_record >> 4) * 512 + l * 16 + (byte_in_record & 15);
  return (byte_in_record >> 3) * 256 + l * 8 + (byte_in_record & 7);
}

// read the code of (token t, channel d) of a group from its bytes (any address space)
TQ_HD int v_get_code(const uint8_t* grp, int bits, int t, int d) {
  int l = v_lane(t, d), p = v_pair(t, d), odd = t & 1;
  if (bits == 4) {
    uint8_t b = grp[v_record_byte_off(4, l, p)];
    return odd ? (b >> 4) : (b & 15);
  }
  int bit = 6 * p + 3 * odd;
  int b0 = grp[v_record_byte_off(3, l, bit >> 3)];
  int b1 = ((bit >> 3) + 1 < 24) ? grp[v_record_byte_off(3, l, (bit >> 3) + 1)] : 0;
  return (((b1 << 8) | b0) >> (bit & 7)) & 7;
}

// ---------------------------------------------------------------------------------------
// element loaders
// ---------------------------------------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<TQ_F32> {
  using type = float;
  static TQ_DEV float ld(const void* p, size_t i) { return ((const float*)p)[i]; }
};
template <>
struct Elem<TQ_F16> {
  using type = __half;
  static TQ_DEV float ld(const void* p, size_t i) { return __half2float(((const __half*)p)[i]); }
};
template <>
struct Elem<TQ_BF16> {
  using type = __nv_bfloat16;
  static TQ_DEV float ld(const void* p, size_t i) {
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
  }
};

TQ_HD int elem_size(int dt) { return dt == TQ_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------------------
constexpr int TQ_PROF_MAX = 4096;
// returns the i-th event of the current call's triple, or nullptr when timing is off/full
cudaEvent_t tq_prof_event(tq_ctx* ctx, int i);
void tq_prof_commit(tq_ctx* ctx);

void tq_set_error(const std::string& msg);
int tq_cuda_fail(cudaError_t e, const char* what);

#define TQ_CUDA(expr)                                      \
  do {                                                     \
    cudaError_t e__ = (expr);                              \
    if (e__ != cudaSuccess) return tq_cuda_fail(e__, #expr); \
  } while (0)

#define TQ_REQUIRE(cond, code, msg) \
  do {                              \
    if (!(cond)) {                  \
      tq_set_error(msg);            \
      return (code);                \
    }                               \
  } while (0)

// kernel launchers implemented in the other translation units ------------------------------
int tq_launch_encode(tq_ctx* ctx, int layer, int seq_begin, int seq_count, const void* k,
                     const void* v, int n_tokens, int64_t seq_stride, int64_t tok_stride,
                     int64_t head_stride, int max_new_blocks, cudaStream_t st);
int tq_launch_decode(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                     int block_end, int with_hot, float* out, float* mlo, cudaStream_t st);
int tq_launch_lse_combine(const float* mlo, int n_parts, int n_rows, int head_dim, float* out,
                          cudaStream_t st);
int tq_launch_dequant(tq_ctx* ctx, int layer, int seq, int start, int end, float* k_out,
                      float* v_out, cudaStream_t st);
size_t tq_mma_scratch_bytes(const tq_geom& g, size_t units);
int tq_launch_clear(tq_ctx* ctx, int layer, int seq_begin, int seq_count, cudaStream_t st);
