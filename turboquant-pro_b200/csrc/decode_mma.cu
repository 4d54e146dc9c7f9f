// Decode-on-codes attention for the common geometry (256-token cold blocks, head_dim 128,
// GQA group 1/2/4/8): a persistent, warp-specialised kernel.
//
//   tiles         stream HBM -> shared memory with bulk asynchronous copies (cp.async.bulk +
//                 mbarrier transaction counts) through a ring of stages; a tile is one cold
//                 page (codes, norms, scales and its outlier list: 34 KB at V3, 38 KB at V4)
//                 or one 32 KB slice of the hot window.  There is no copy warp: the group
//                 that has finished with a stage starts the copy of the tile that uses the
//                 stage next.
//   consumer      groups of four warps; group i owns tiles i, i + NG, i + 2 NG ... of the CTA's
//   groups        share, so NG pages are being worked on at once while the next ones land.
//                 Per page a group first builds the query- and page-dependent operands
//                 (w = q * scale split into fp16 hi/lo tensor-core fragments, bias = q . mean,
//                 the per-token outlier corrections: each warp for its own 64 tokens), then
//                 each warp attends its 64 tokens: 4-bit key codes and 3/4-bit value code
//                 pairs become fp16 pairs through one conflict-free shared-memory table
//                 lookup each and go straight into m16n8k16 tensor-core tiles as register
//                 fragments (scores: M = 16 tokens, N = four query heads x {hi, lo} weight
//                 parts, K = 16 channels; values: M = 16 channels, N = the same eight columns,
//                 K = 16 tokens; the probabilities change from the score tile's layout to the
//                 value tile's with one 8x8 register transpose); online softmax in fp32
//                 registers.  K and V are never materialised.
//
// Work is a flat list of tiles over all (sequence, KV head) units of the layer, cut into
// equal contiguous shares, one per CTA (one CTA per SM), so ragged contexts balance.
// Every consumer warp keeps its own softmax state; when a group leaves a unit its four warps
// merge their states and write one partial (m, l, acc[D]); the combine kernel merges the
// partials in a fixed order and applies the single inverse rotation of the value accumulator.
//
// All waits are bounded: a wait that runs out sets bit 1 of the status word and an abort
// flag that makes every later wait return at once, so the kernel always terminates.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "xchg.cuh"

namespace {

#ifndef TQ_GW
#define TQ_GW 4
#endif
// warps per consumer group: 4 (three groups, 168 registers per thread); 8 (two groups, 128
// registers) builds and runs but measured 30 % slower on the common geometry
constexpr int GW = TQ_GW;
constexpr int TPW = 256 / GW;        // tokens of a cold page per warp
constexpr int HALVES = TPW / 16;     // 16-token tiles per warp and page
static_assert(GW == 4 || GW == 8, "a warp owns 64 or 32 tokens of a page");
constexpr int MAX_NG = 3;            // most consumer groups
constexpr int MAX_UNITS = 512;       // (sequence, KV head) units per launch; larger layers take several
constexpr int BLK = 256;             // tokens per cold page
constexpr float NEG_BIG = -1.0e30f;
constexpr int SPIN_LIMIT = 1 << 18;  // default probes per wait; each may suspend up to ~2 us

struct MmaArgs {
  tq_geom g;
  const uint8_t* pages;
  const uint8_t* hot_k;
  const uint8_t* hot_v;
  const uint32_t* pool_dec;
  const int32_t* seq_len;
  const Tables* tables;
  const void* q;
  float* partials;
  int* plan_g;  // {T, Q, P[0..n_units], nb[0..n_units)} published by CTA 0 for the combine
  float* out;
  float* mlo;
  int32_t* status;
  unsigned long long* trace;  // optional: SM clock stamps of CTA 0's first 64 tiles
  int layer, q_dtype, n_units, n_cta;
  int unit_base;  // first unit of the layer this launch covers (a multiple of the KV head count)
  int use_tmap;  // 16-bit hot tiles arrive through the tensor maps, 128-byte swizzled
  int n_groups;  // consumer groups of the attention kernel (the combine enumerates their slots)
  int block_begin, block_end, with_hot;
  int spin_limit;     // probes a bounded wait makes before it gives up
  int withhold_tile;  // test hook: CTA 0 never starts the copy of this tile of its share (-1: off)
  float scale_log2;
  // Sequence split over several GPUs: the merge kernel hands its rows to the other ranks and
  // merges theirs itself (xchg_on), instead of writing the states for a separate exchange.
  int xchg_on;
  XchgDev xchg;
};

// ---- PTX helpers --------------------------------------------------------------------------
TQ_DEV uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

TQ_DEV void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
TQ_DEV void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
TQ_DEV void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// one bounded, possibly suspending probe of a barrier phase (the hint caps the suspension)
TQ_DEV uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok;
}
// plain, non-multicast bulk copy from this GPU's global memory into this CTA's shared memory
TQ_DEV void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Read of a constant lookup table: not volatile, so the scheduler may move and overlap it
// freely (the tables never change after the prologue's barrier).
TQ_DEV uint32_t lut_ld(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
TQ_DEV void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2-D tile of a tensor map into shared memory (no multicast); x counts elements of the inner
// dimension (x * 2 bytes is a multiple of 16 at every call site), y rows
TQ_DEV void tensor_g2s(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// four 8x8 matrices of 16-bit elements, rows given by the lanes' addresses (lanes 8m..8m+7:
// matrix m); thread (r, c) receives row r, columns 2c and 2c+1 of each, or with `trans`
// rows 2c and 2c+1 of column r
TQ_DEV void ldsm_x4(uint32_t* v, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(addr)
               : "memory");
}
TQ_DEV void ldsm_x4_trans(uint32_t* v, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(addr)
               : "memory");
}
// transpose of an 8x8 matrix of 16-bit elements held one row per four lanes (lane 4i + c:
// row i, columns 2c and 2c+1)
TQ_DEV uint32_t transpose8x8(uint32_t v) {
  uint32_t o;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(o) : "r"(v));
  return o;
}
// 2^x in one instruction (denormal results flush to zero; arguments here are <= 0 or tiny)
TQ_DEV float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
TQ_DEV uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *(uint32_t*)&h;
}
// two bf16 in one word -> two fp16 in one word (exact for magnitudes in fp16 range)
TQ_DEV uint32_t bf16x2_to_h2(uint32_t w) {
  return pack_h2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// ---- shared-memory plan --------------------------------------------------------------------
// [value table (8 KB aligned at V3) | key table | plan | group scratch x NG | barriers |
//  stages].  A stage holds one tile; a group's scratch holds its query copy, the fragments
// and bias of the page it works on and one outlier-correction strip per warp.
template <int G, int VB, int NG>
struct SmemT {
  // a tile is a whole page (34816 B at V3, 38912 B at V4) or 32 KB of hot rows
  static constexpr int DATA_BYTES = VB == 3 ? 34816 : 38912;
  static constexpr int LUTK_BYTES = 256 * 128;
  static constexpr int LUTV_BYTES = (VB == 3 ? 64 : 256) * 128;
  // the 3-bit value table starts on an 8 KB boundary (its addresses are formed with OR)
  static constexpr int ALIGN_SLACK = VB == 3 ? 8192 : 0;
  static constexpr int PLAN_BYTES = 8192;
  static constexpr int QC_BYTES = TQ_D * G * 4;  // [128][G] query values
  static constexpr int FRAG_BYTES = 8 * 32 * 16;  // [G/4 column groups][8 k-steps][32 lanes] x 8 B
  static constexpr int BIAS_BYTES = 8 * GW * 4 + 128;  // [8 heads][GW]: a partial per warp (+ spare)
  static constexpr int CORR_STRIDE = TPW + 8;    // floats per query row: rows on different banks
  static constexpr int CORR_BYTES = G * CORR_STRIDE * 4;  // per warp
  static constexpr int FRAG_OFF = QC_BYTES;
  static constexpr int BIAS_OFF = FRAG_OFF + FRAG_BYTES;
  static constexpr int CORR_OFF = BIAS_OFF + BIAS_BYTES;
  static constexpr int GROUP_BYTES = CORR_OFF + GW * CORR_BYTES;
  // the stages start on a 1 KB boundary (the swizzled hot tiles need it)
  static constexpr int BARS_BYTES = 256 + (1024 - (NG * GROUP_BYTES + 256) % 1024) % 1024;
  static constexpr int FIXED =
      ALIGN_SLACK + LUTK_BYTES + LUTV_BYTES + PLAN_BYTES + NG * GROUP_BYTES + BARS_BYTES;
  static constexpr int FIT = (232448 - FIXED) / DATA_BYTES;
  static constexpr int NSTAGE = FIT >= 4 ? 4 : FIT;
  static constexpr int TOTAL = FIXED + NSTAGE * DATA_BYTES;
};

// three groups when four stages still fit beside them (one page always in flight), else two
template <int G, int VB>
struct Cfg {
  static constexpr int NG = GW == 8 ? 2 : (SmemT<G, VB, 3>::NSTAGE >= 4 ? 3 : 2);
  using SM = SmemT<G, VB, NG>;
  static_assert(SM::NSTAGE > NG, "a group refills a stage for a later tile of another group");
  static constexpr int CWT = NG * GW;  // consumer warps
  static constexpr int THREADS = CWT * 32;
};

struct Plan {  // lives in shared memory
  int P[MAX_UNITS + 1];      // prefix sums of tiles per unit
  int hot_start[MAX_UNITS];  // first hot token position of each unit's sequence
  short nb[MAX_UNITS];       // cold tiles of each unit
  short b0[MAX_UNITS];       // first cold block attended
  short hot_len[MAX_UNITS];  // hot tokens attended
};

struct Tile {
  int u, kind, idx;  // kind 0: cold page `idx` (absolute block), 1: hot tile `idx`
};

TQ_DEV int hot_tile_tokens(int dt) { return dt == TQ_F32 ? 32 : 64; }

// cold / hot tile counts of a unit, identical in the attention and the combine kernel
TQ_DEV void unit_tiles(const MmaArgs& a, int unit, int& nb, int& ht, int& b0, int& hot_start,
                       int& hot_len) {
  const tq_geom& g = a.g;
  const int seq = (a.unit_base + unit) / g.n_kv_heads;
  const int N = a.seq_len[a.layer * g.n_seqs + seq];
  const int nbt = n_cold_blocks(N, g.hot_window, BLK);
  b0 = min(a.block_begin, nbt);
  const int b1 = a.block_end < 0 ? nbt : min(a.block_end, nbt);
  nb = max(b1 - b0, 0);
  hot_start = nbt * BLK;
  hot_len = a.with_hot ? N - nbt * BLK : 0;
  const int htt = hot_tile_tokens(g.kv_dtype);
  ht = (hot_len + htt - 1) / htt;
}

// Fills the plan; every thread of the CTA must call it.  `scratch` takes the chunk totals of
// the scan (16 x 8 bytes) and, from byte 256 on, nbp[0 .. n_units]: the prefix sums of the
// units' cold tiles (tile positions + cold tiles before them = the cost a CTA's share is cut by).
TQ_DEV void build_plan(const MmaArgs& a, Plan* plan, void* scratch, int tid, int nthreads) {
  unsigned long long* tot = (unsigned long long*)scratch;
  int* nbp = (int*)scratch + 64;
  for (int u = tid; u < a.n_units; u += nthreads) {
    int nb, ht, b0, hs, hl;
    unit_tiles(a, u, nb, ht, b0, hs, hl);
    plan->nb[u] = (short)nb;
    plan->b0[u] = (short)b0;
    plan->hot_start[u] = hs;
    plan->hot_len[u] = (short)hl;
    plan->P[u + 1] = nb + ht;  // tiles of the unit, scanned below
  }
  __syncthreads();
  // inclusive scan: every warp scans chunks of 32 units, then the chunk totals are added
  const int lane = tid & 31, n_chunks = (a.n_units + 31) / 32;
  for (int ch = tid >> 5; ch < n_chunks; ch += nthreads >> 5) {
    const int i = 32 * ch + lane;
    // tiles in the low word, cold tiles in the high word: one scan for both
    unsigned long long v = i < a.n_units ? (unsigned long long)(unsigned)plan->P[i + 1] |
                                               ((unsigned long long)(unsigned)plan->nb[i] << 32)
                                         : 0ull;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    if (i < a.n_units) {
      plan->P[i + 1] = (int)(unsigned)v;
      nbp[i + 1] = (int)(v >> 32);
    }
    if (lane == 31) tot[ch] = v;
  }
  if (tid == 0) {
    plan->P[0] = 0;
    nbp[0] = 0;
  }
  __syncthreads();
  for (int i = tid; i < a.n_units; i += nthreads) {
    unsigned long long base = 0;
    for (int ch = 0; ch < (i >> 5); ++ch) base += tot[ch];
    plan->P[i + 1] += (int)(unsigned)base;
    nbp[i + 1] += (int)(base >> 32);
  }
  __syncthreads();
}

// First tile of the share that starts at cost `v`.  A cold tile costs two units and a hot
// tile one (a hot tile takes about half the time of a page), so unit u spans the costs
// P[u] + nbp[u] .. P[u+1] + nbp[u+1] and a tile belongs to the share its first unit falls in.
TQ_DEV int tile_at_cost(const Plan* plan, const int* nbp, int n_units, int v) {
  if (v >= plan->P[n_units] + nbp[n_units]) return plan->P[n_units];
  int lo = 0, hi = n_units - 1;  // largest u whose first cost is <= v
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (plan->P[mid] + nbp[mid] <= v) lo = mid; else hi = mid - 1;
  }
  const int local = v - (plan->P[lo] + nbp[lo]), nb = plan->nb[lo];
  return plan->P[lo] + (local < 2 * nb ? (local + 1) >> 1 : local - nb);
}

TQ_DEV int find_unit(const Plan* plan, int n_units, int pos) {
  int lo = 0, hi = n_units - 1;  // largest u with P[u] <= pos
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (plan->P[mid] <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// debugging aid: slot k of tile t gets the SM clock (CTA 0, first 64 tiles, one lane)
#define TQ_TRACE(k)                                                     \
  do {                                                                  \
    if (a.trace != nullptr && blockIdx.x == 0 && lane == 0 && t < 63)   \
      a.trace[t * 8 + (k)] = (unsigned long long)clock64();             \
  } while (0)
// row 63 of the trace: the kernel's own phases (entry, tables built, predecessor done, plan
// built, first copies started), stamped by thread 0 of CTA 0
#define TQ_TRACE_PHASE(k)                                               \
  do {                                                                  \
    if (a.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0)      \
      a.trace[63 * 8 + (k)] = (unsigned long long)clock64();            \
  } while (0)

struct Waiter {
  volatile int* abort_flag;
  int32_t* status;
  int limit;
  TQ_DEV void wait(uint32_t bar, uint32_t parity) const {
    for (int i = 0; i < limit; ++i) {
      if (mbar_try(bar, parity)) return;
      if ((i & 15) == 15 && *abort_flag) return;
    }
    *abort_flag = 1;
    atomicOr(status, TQ_STATUS_WAIT_TIMEOUT);
  }
  // bounded wait that ignores the abort flag
  TQ_DEV void drain(uint32_t bar, uint32_t parity) const {
    for (int i = 0; i < limit; ++i)
      if (mbar_try(bar, parity)) return;
  }
};

// fp16 hi / lo fragments of four consecutive weights of a row: {hi01, lo01, hi23, lo23}
TQ_DEV uint4 frag_hilo(float w0, float w1, float w2, float w3) {
  __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
  float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
  uint4 o;
  o.x = *(uint32_t*)&h01;
  o.y = pack_h2(w0 - f01.x, w1 - f01.y);
  o.z = *(uint32_t*)&h23;
  o.w = pack_h2(w2 - f23.x, w3 - f23.y);
  return o;
}

template <int G, int VB>
__global__ void __launch_bounds__(Cfg<G, VB>::THREADS, 1)
    decode_mma_kernel(MmaArgs a, const __grid_constant__ CUtensorMap tm_hot_k,
                      const __grid_constant__ CUtensorMap tm_hot_v) {
  using CF = Cfg<G, VB>;
  using SM = typename CF::SM;
  constexpr int NG = CF::NG, NSTAGE = SM::NSTAGE, CWT = CF::CWT, THREADS = CF::THREADS;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const tq_geom& g = a.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;

  // the 3-bit value table sits on an 8 KB boundary of the shared address space so that a
  // table address is (index bits) | (base + lane offset), one logic instruction
  uint8_t* smem = smem_raw;
  if (VB == 3) smem += (8192u - (smem_addr(smem_raw) & 8191u)) & 8191u;
  uint8_t* lutv_p = smem;
  uint8_t* lutk_p = lutv_p + SM::LUTV_BYTES;
  Plan* plan = (Plan*)(lutk_p + SM::LUTK_BYTES);
  static_assert(sizeof(Plan) <= SM::PLAN_BYTES - 64, "plan does not fit its shared-memory slot");
  // NF4[c] - fp16(NF4[c]): what the half-precision key table loses, added back in float32
  // for the widest channels of a page
  float* dtab = (float*)((uint8_t*)plan + SM::PLAN_BYTES - 64);
  uint8_t* groups = (uint8_t*)plan + SM::PLAN_BYTES;
  // "tile landed" barriers.  Tile t lands in stage t % NSTAGE but signals barrier
  // t % (2 NSTAGE): stages are refilled out of order (by whichever group frees them), so a
  // group can come to wait for tile t + NSTAGE while tile t - NSTAGE still occupies the
  // stage; with one barrier per stage that wait would see the parity of the older phase.
  uint64_t* bars = (uint64_t*)(groups + NG * SM::GROUP_BYTES);
  volatile int* abort_flag = (volatile int*)(bars + 16);
  uint8_t* stages = (uint8_t*)bars + SM::BARS_BYTES;
  static_assert(2 * NSTAGE <= 16, "barrier slots");

  TQ_TRACE_PHASE(0);
  const uint32_t full0 = smem_addr(bars);
  if (tid == 0) {
    for (int s = 0; s < 2 * NSTAGE; ++s) mbar_init(full0 + 8 * s, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // lookup tables: entry-major, one copy per lane so that a warp's 32 lookups never collide
  {
    float* small = (float*)groups;  // 32 floats of scratch until the groups claim the area
    if (tid < 16) small[tid] = a.tables->grid[tid];
    else if (tid < 32) small[tid] = a.tables->centroids[tid - 16];
    __syncthreads();
    if (tid < 16) dtab[tid] = small[tid] - __half2float(__float2half_rn(small[tid]));
    // an entry is one word repeated 32 times (a copy per lane): a thread computes the word of
    // its entries once and stores it as eight 16-byte vectors
    constexpr int NV = VB == 3 ? 64 : 256;
    for (int en = tid; en < 256 + NV; en += THREADS) {
      uint32_t w;
      uint4* dst;
      if (en < 256) {
        w = pack_h2(small[en & 15], small[en >> 4]);
        dst = (uint4*)lutk_p + en * 8;
      } else {
        const int b = en - 256;
        const int ca = VB == 3 ? (b & 7) : (b & 15), cb = VB == 3 ? (b >> 3) : (b >> 4);
        w = pack_h2(small[16 + ca], small[16 + cb]);
        dst = (uint4*)lutv_p + b * 8;
      }
      const uint4 w4 = make_uint4(w, w, w, w);
      // (the lanes of a warp write different 16-byte columns of their 128-byte entries in
      // every step, which spreads a store over all banks)
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[(i + lane) & 7] = w4;
    }
  }
  // Both kernels of a decode call are launched with programmatic stream serialization: this
  // one may start while the kernel before it in the stream is still running.  Up to here it
  // has read only the constant tables; everything else (lengths, query, pages, scratch) is
  // touched after the wait, which returns once that kernel has completed.
  TQ_TRACE_PHASE(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  TQ_TRACE_PHASE(2);
  // (contains the __syncthreads that publish all of the above; the groups' area is free)
  build_plan(a, plan, groups, tid, THREADS);
  // the combine kernel that follows may be scheduled wherever an SM frees up
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // The tile list is cut into shares of equal cost (cold tile 2, hot tile 1), one per CTA.
  const int* nbp = (const int*)groups + 64;
  const int VT = plan->P[a.n_units] + nbp[a.n_units];
  const int Q = (VT + a.n_cta - 1) / a.n_cta;
  const int lo = tile_at_cost(plan, nbp, a.n_units, min((int)blockIdx.x * Q, VT));
  const int hi = tile_at_cost(plan, nbp, a.n_units, min((int)(blockIdx.x + 1) * Q, VT));
  if (blockIdx.x == 0) {  // the combine kernel reads the plan instead of rebuilding it
    if (tid == 0) a.plan_g[0] = a.n_cta;
    for (int u = tid; u <= a.n_units; u += THREADS) a.plan_g[2 + u] = plan->P[u];
    for (int u = tid; u < a.n_units; u += THREADS) a.plan_g[3 + a.n_units + u] = plan->nb[u];
    // ... and where every CTA's share starts
    for (int i = tid; i <= a.n_cta; i += THREADS)
      a.plan_g[3 + 2 * a.n_units + i] = tile_at_cost(plan, nbp, a.n_units, min(i * Q, VT));
  }
  __syncthreads();  // the cold-tile sums lie in the area the groups take over now
  if (lo >= hi) return;
  TQ_TRACE_PHASE(3);
  const Waiter waiter{abort_flag, a.status, a.spin_limit};
  const int htt = hot_tile_tokens(g.kv_dtype);
  const int esz = elem_size(g.kv_dtype);

  // A cursor into the tile list: the unit that holds a position, kept in registers and looked
  // up again only when the positions (which only grow) leave the unit.
  struct Cursor {
    int u, P0, P1, nb, b0;
  };
  auto tile_at = [&](int pos, Cursor& cu) -> Tile {
    if (pos >= cu.P1) {
      int u = cu.u;
      while (pos >= plan->P[u + 1]) ++u;
      cu.u = u;
      cu.P0 = plan->P[u];
      cu.P1 = plan->P[u + 1];
      cu.nb = plan->nb[u];
      cu.b0 = plan->b0[u];
    }
    Tile t;
    t.u = cu.u;
    const int j = pos - cu.P0;
    t.kind = j >= cu.nb;
    t.idx = t.kind == 0 ? cu.b0 + j : j - cu.nb;
    return t;
  };
  // units of this layer are numbered (sequence, KV head) row-major, and so are their pages,
  // hot rings, pool lists and query rows: no division by the head count is ever needed
  const size_t unit0 = (size_t)a.layer * g.n_seqs * g.n_kv_heads + a.unit_base;

  // The copy of tile t of this CTA's share: describe() works out addresses and sizes (it can
  // run before the stage is free), fire() starts it (the stage must be free: never used, or
  // the caller's group has just finished with it).
  struct CopyDesc {
    const uint8_t* src;
    const uint8_t* src2;  // second source of a hot tile (the value rows), else null
    uint32_t bytes, dst, bar;
    int row;  // hot tile: its first row in the ring seen as one 2-D array
    int t;    // index of the tile in the CTA's share
  };
  const int total = hi - lo;
  auto describe = [&](int t, Cursor& cu) -> CopyDesc {
    const Tile tl = tile_at(lo + t, cu);
    const size_t unit = unit0 + tl.u;
    CopyDesc d;
    d.t = t;
    d.dst = smem_addr(stages + (size_t)(t % NSTAGE) * SM::DATA_BYTES);
    d.bar = full0 + 8 * (t % (2 * NSTAGE));
    if (tl.kind == 0) {
      d.src = a.pages + (unit * g.max_blocks + tl.idx) * (size_t)g.page_bytes;
      d.src2 = nullptr;
      d.bytes = (uint32_t)g.page_bytes;
    } else {
      const int slot = (plan->hot_start[tl.u] + tl.idx * htt) % g.hot_cap;
      const size_t off = (unit * g.hot_cap + slot) * (size_t)(TQ_D * esz);
      d.src = a.hot_k + off;
      d.src2 = a.hot_v + off;
      d.bytes = (uint32_t)(htt * TQ_D * esz);
      d.row = (int)(unit * g.hot_cap) + slot;
    }
    return d;
  };
  int last_fired = -1;  // the latest tile whose copy this thread started
  auto fire = [&](const CopyDesc& d) {
    // (test hook: a withheld copy leaves its barrier incomplete, so the wait for it runs out)
    if (blockIdx.x == 0 && d.t == a.withhold_tile) return;
    last_fired = d.t;
    if (d.src2 == nullptr) {
      mbar_arrive_expect_tx(d.bar, d.bytes);
      bulk_g2s(d.dst, d.src, d.bytes, d.bar);
    } else if (a.use_tmap) {
      // 64 rows x 64 channels per copy, each landing as 8 KB of 128-byte rows whose 16-byte
      // chunks are XOR-swizzled with the row number: [K left | K right | V left | V right]
      mbar_arrive_expect_tx(d.bar, 2 * d.bytes);
      tensor_g2s(d.dst, &tm_hot_k, 0, d.row, d.bar);
      tensor_g2s(d.dst + 8192, &tm_hot_k, 64, d.row, d.bar);
      tensor_g2s(d.dst + 16384, &tm_hot_v, 0, d.row, d.bar);
      tensor_g2s(d.dst + 24576, &tm_hot_v, 64, d.row, d.bar);
    } else {
      mbar_arrive_expect_tx(d.bar, 2 * d.bytes);
      bulk_g2s(d.dst, d.src, d.bytes, d.bar);
      bulk_g2s(d.dst + d.bytes, d.src2, d.bytes, d.bar);
    }
  };

  // ============================== consumer groups ============================================
  const int gi = warp / GW, gw = warp % GW, gtid = tid - gi * (GW * 32);
  const int u_first = find_unit(plan, a.n_units, lo);
  Cursor u_iss = {u_first, 0, 0, 0, 0};  // cursor of the copies this thread starts
  if (warp == 0 && lane < min(NSTAGE, total)) fire(describe(lane, u_iss));  // a lane per tile
  TQ_TRACE_PHASE(4);
  uint8_t* gs = groups + gi * SM::GROUP_BYTES;
  float* qc = (float*)gs;  // [128][G]; a group of eight as two planes of [128][4]
  // (a correction's two 16-byte loads of a row then spread over all eight 16-byte bank
  // groups instead of four)
  constexpr int QP = G == 8 ? 4 : G;  // heads per plane
  auto qi = [&](int row, int h) -> int { return G == 8 ? (h >> 2) * (TQ_D * 4) + row * 4 + (h & 3) : row * G + h; };
  uint2* frag = (uint2*)(gs + SM::FRAG_OFF);                // [G/4][8 k-steps][32 lanes]
  float* bias_s = (float*)(gs + SM::BIAS_OFF);              // [8 heads][GW]
  float* corr_w = (float*)(gs + SM::CORR_OFF) + gw * (G * SM::CORR_STRIDE);  // this warp's strip
  auto group_sync = [&]() {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "n"(GW * 32) : "memory");
  };

  const uint32_t lutk = smem_addr(lutk_p) + lane * 4;
  const uint32_t lutv = smem_addr(lutv_p) + lane * 4;  // 8 KB aligned base | lane offset
  // Column n of a score or value tile: query head n / 2, and n & 1 selects the hi or lo fp16
  // part of its weights.  A group of eight heads takes two such score tiles (heads 0-3, 4-7);
  // its value tile then has head n / 2 + 4 (n & 1) in column n.  A lane's two columns (2c,
  // 2c+1) therefore always belong to head c (and c + 4): its softmax state is its own.
  constexpr int NH = G == 8 ? 2 : 1;
  int hc[NH];  // the lane's heads, clamped to the group
#pragma unroll
  for (int nh = 0; nh < NH; ++nh) hc[nh] = min(c + 4 * nh, G - 1);
  float m_run[NH], l_run[NH];  // l_run: the sum over this lane's own tokens
  float acc[8][4];
  auto reset_state = [&]() {
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      m_run[nh] = NEG_BIG;
      l_run[nh] = 0.0f;
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
  };
  reset_state();

  // Writes the group's partial (m, l, acc[D]) of one (unit, kind): the four warps merge their
  // states through shared memory (the fragment / bias / correction areas are idle between
  // tiles) and the 128 threads store one coalesced record.  Called by all warps of the group.
  auto flush = [&](int u, int kind) {
    // as many warps at a time as there is room for accumulator copies (row stride 136
    // floats: the cold layout then stores without bank conflicts)
    constexpr int MG_STRIDE = TQ_D + 8, MG_ONE = G * MG_STRIDE * 4;
    constexpr int MG_ROOM = SM::GROUP_BYTES - SM::FRAG_OFF - 2 * GW * 8 * 4;
    constexpr int MG_PAR = MG_ROOM >= 4 * MG_ONE ? 4 : (MG_ROOM >= 2 * MG_ONE ? 2 : 1);
    static_assert(MG_ROOM >= MG_ONE, "merge scratch");
    float* mg_m = (float*)(gs + SM::FRAG_OFF);  // [GW][8] maxima of the warps, per query row
    float* mg_l = mg_m + GW * 8;                // [GW][8] their sums
    float* mg_acc = mg_l + GW * 8;              // [MG_PAR][G][MG_STRIDE] scaled accumulators
    group_sync();  // every warp has finished its last tile
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      float l = l_run[nh];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      if (r == 0) {
        mg_m[gw * 8 + c + 4 * nh] = m_run[nh];
        mg_l[gw * 8 + c + 4 * nh] = l;
      }
    }
    group_sync();
    float f[NH];  // this warp's state relative to the group's maximum, per head of the lane
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      float M = NEG_BIG;
#pragma unroll
      for (int w = 0; w < GW; ++w) M = fmaxf(M, mg_m[w * 8 + c + 4 * nh]);
      f[nh] = exp2f(mg_m[gw * 8 + c + 4 * nh] - M);
    }
    float* mine = mg_acc + (gw % MG_PAR) * (G * MG_STRIDE);
    for (int step = 0; step < GW / MG_PAR; ++step) {
      if (gw / MG_PAR == step) {
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int d = (kind == 0 || a.use_tmap) ? 16 * mt + r + 8 * x : 16 * r + 2 * mt + x;
            if (G == 8) {  // the two columns are two heads
#pragma unroll
              for (int y = 0; y < 2; ++y) {
                const float v = acc[mt][2 * x + y] * f[NH - 1 < y ? NH - 1 : y];
                float* dst = mine + (c + 4 * y) * MG_STRIDE + d;
                if (step == 0) *dst = v; else *dst += v;
              }
            } else if (c < G) {  // ... or the hi and lo parts of one head's probabilities
              const float v = (acc[mt][2 * x] + acc[mt][2 * x + 1]) * f[0];
              float* dst = mine + c * MG_STRIDE + d;
              if (step == 0) *dst = v; else *dst += v;
            }
          }
      }
      group_sync();
    }
    float* pp = a.partials +
                ((((size_t)u + blockIdx.x) * 2 + kind) * NG + gi) * (size_t)(G * TQ_PART_STRIDE);
    if (gtid < TQ_D) {
#pragma unroll
      for (int gg = 0; gg < G; ++gg) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < MG_PAR; ++w) v += mg_acc[(w * G + gg) * MG_STRIDE + gtid];
        pp[gg * TQ_PART_STRIDE + 2 + gtid] = v;
      }
    }
    if (gtid < G) {
      float M = NEG_BIG, L = 0.0f;
#pragma unroll
      for (int w = 0; w < GW; ++w) M = fmaxf(M, mg_m[w * 8 + gtid]);
#pragma unroll
      for (int w = 0; w < GW; ++w) L += mg_l[w * 8 + gtid] * exp2f(mg_m[w * 8 + gtid] - M);
      pp[gtid * TQ_PART_STRIDE] = M;
      pp[gtid * TQ_PART_STRIDE + 1] = L;
    }
  };

  // online-softmax update with the scores of this lane's two tokens (rows r and r + 8 of a
  // 16-token tile) for each of its heads; leaves the probabilities in sv
  auto softmax16 = [&](float (&sv)[NH][2], const bool (&ok)[2]) {
    float cf[NH];
    bool grew = false;
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      float mx = fmaxf(ok[0] ? sv[nh][0] : NEG_BIG, ok[1] ? sv[nh][1] : NEG_BIG);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[nh], mx);
      cf[nh] = ex2(m_run[nh] - m_new);
      sv[nh][0] = ok[0] ? ex2(sv[nh][0] - m_new) : 0.0f;
      sv[nh][1] = ok[1] ? ex2(sv[nh][1] - m_new) : 0.0f;
      l_run[nh] = l_run[nh] * cf[nh] + (sv[nh][0] + sv[nh][1]);
      grew |= m_new > m_run[nh];
      m_run[nh] = m_new;
    }
    if (__any_sync(0xffffffffu, grew)) {
      const float f0 = cf[0], f1 = cf[NH - 1];
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        acc[mt][0] *= f0;
        acc[mt][1] *= f1;
        acc[mt][2] *= f0;
        acc[mt][3] *= f1;
      }
    }
  };
  // the same over NT consecutive 16-token tiles at once (all tokens valid): one reduction
  // and at most one rescaling of the accumulator for all of them
  auto softmax_many = [&](auto& sv) {
    constexpr int NT = sizeof(sv) / sizeof(sv[0]);
    float cf[NH];
    bool grew = false;
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      float mx = NEG_BIG;
#pragma unroll
      for (int h = 0; h < NT; ++h) mx = fmaxf(mx, fmaxf(sv[h][nh][0], sv[h][nh][1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[nh], mx);
      cf[nh] = ex2(m_run[nh] - m_new);
      float sum = 0.0f;
#pragma unroll
      for (int h = 0; h < NT; ++h) {
        sv[h][nh][0] = ex2(sv[h][nh][0] - m_new);
        sv[h][nh][1] = ex2(sv[h][nh][1] - m_new);
        sum += sv[h][nh][0] + sv[h][nh][1];
      }
      l_run[nh] = l_run[nh] * cf[nh] + sum;
      grew |= m_new > m_run[nh];
      m_run[nh] = m_new;
    }
    if (__any_sync(0xffffffffu, grew)) {
      const float f0 = cf[0], f1 = cf[NH - 1];
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        acc[mt][0] *= f0;
        acc[mt][1] *= f1;
        acc[mt][2] *= f0;
        acc[mt][3] *= f1;
      }
    }
  };
  // The value tile's B fragments (tokens down the K dimension, the eight columns across) from
  // the probabilities of this lane's tokens, already times the token's value norm: column 2c
  // gets head c and column 2c+1 the rounding residual of the same number (so the product is
  // accurate beyond fp16), or head c + 4 for a group of eight.
  auto prob_frags = [&](const float (&sv)[NH][2], float n0, float n1, uint32_t& pb0,
                        uint32_t& pb1) {
    uint32_t w0, w1;
    if (G == 8) {
      w0 = pack_h2(sv[0][0] * n0, sv[NH - 1][0] * n0);
      w1 = pack_h2(sv[0][1] * n1, sv[NH - 1][1] * n1);
    } else {
      const float v0 = sv[0][0] * n0, v1 = sv[0][1] * n1;
      const float h0 = __half2float(__float2half_rn(v0)), h1 = __half2float(__float2half_rn(v1));
      w0 = pack_h2(h0, v0 - h0);
      w1 = pack_h2(h1, v1 - h1);
    }
    pb0 = transpose8x8(w0);  // tokens 0-7 of the tile: lane (r, c) gets tokens 2c, 2c+1, column r
    pb1 = transpose8x8(w1);  // tokens 8-15
  };

  Cursor u_cur = {u_first, 0, 0, 0, 0};
  int cur_u = -1, cur_kind = -1, q_unit = -1;
  for (int pos = lo + gi; pos < hi; pos += NG) {
    const int t = pos - lo, s = t % NSTAGE;
    const uint32_t full_bar = full0 + 8 * (t % (2 * NSTAGE));
    const uint32_t full_par = (t / (2 * NSTAGE)) & 1;
    const Tile tl = tile_at(pos, u_cur);
    if (tl.u != cur_u || tl.kind != cur_kind) {
      if (cur_u >= 0) flush(cur_u, cur_kind);
      reset_state();
      cur_u = tl.u;
      cur_kind = tl.kind;
    }
    // The stage of the group's previous tile is refilled once all four warps are done with
    // it; the warps take turns at starting the copy and describe it before the barrier.
    const bool refill = lane == 0 && gw == (t / NG) % GW && t >= NG && t - NG + NSTAGE < total;
    CopyDesc cd;
    if (refill) cd = describe(t - NG + NSTAGE, u_iss);
    // the group is done with the fragments, bias, query copy and stage of its previous tile
    group_sync();
    if (refill && !*abort_flag) {
      fire(cd);
      TQ_TRACE(1);
    }
    if (tl.u != q_unit) {  // new unit: reload its query rows
      q_unit = tl.u;
      if (gtid < TQ_D) {
        // thread d of the group loads channel d of the G rows: coalesced, independent loads.
        // The softmax scale (1/sqrt(D), in the log2 domain) rides on the query, so scores,
        // bias and corrections come out already scaled.
        // query heads follow their KV head
        const size_t q0 = (size_t)(a.unit_base + tl.u) * (G * TQ_D) + gtid;
        float qv[G];
        if (a.q_dtype == TQ_F32) {
#pragma unroll
          for (int rr = 0; rr < G; ++rr) qv[rr] = ((const float*)a.q)[q0 + rr * TQ_D];
        } else if (a.q_dtype == TQ_F16) {
#pragma unroll
          for (int rr = 0; rr < G; ++rr)
            qv[rr] = __half2float(((const __half*)a.q)[q0 + rr * TQ_D]);
        } else {
#pragma unroll
          for (int rr = 0; rr < G; ++rr)
            qv[rr] = __bfloat162float(((const __nv_bfloat16*)a.q)[q0 + rr * TQ_D]);
        }
#pragma unroll
        for (int rr = 0; rr < G; ++rr) qc[qi(q_row(gtid), rr)] = a.scale_log2 * qv[rr];
      }
      group_sync();
    }
    const uint8_t* st = stages + (size_t)s * SM::DATA_BYTES;
    if (warp == 0) TQ_TRACE(2);
    waiter.wait(full_bar, full_par);
    if (warp == 0) TQ_TRACE(3);

    // ---- operands that depend on the query and the page ------------------------------------
    const bool cold = tl.kind == 0;
    const float* scale = (const float*)(st + g.scale_off);
    {
      // B fragments of the weights: lane (r, c) holds column r (head r / 2, part r & 1) at the
      // channels of rows 2c, 2c+1 and 2c+8, 2c+9 of the k-step
      const float* mean = (const float*)(st + g.mean_off);
      float bias[NH];
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) bias[nh] = 0.0f;
#pragma unroll
      for (int i = 0; i < 8 / GW; ++i) {  // this warp's k-steps
        const int j = gw + GW * i;
        // channels of this lane's four fragment values: pages order them 32c + 4j + i (the
        // order of their code bytes); swizzled hot tiles are read by 8x8 matrix loads and keep
        // the tensor-core tile's own order 16j + {2c, 2c+1, 2c+8, 2c+9}
        const int d0 = 32 * c + 4 * j, dn = 16 * j + 2 * c;
        const bool natural = !cold && a.use_tmap;
        float4 s4 = make_float4(1.f, 1.f, 1.f, 1.f), m4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cold) {
          s4 = *(const float4*)&scale[d0];
          m4 = *(const float4*)&mean[d0];
        }
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
          const int hb = 4 * nh + (r >> 1);
          float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (hb < G) {
            q4.x = qc[qi(q_row(natural ? dn : d0 + 0), hb)];
            q4.y = qc[qi(q_row(natural ? dn + 1 : d0 + 1), hb)];
            q4.z = qc[qi(q_row(natural ? dn + 8 : d0 + 2), hb)];
            q4.w = qc[qi(q_row(natural ? dn + 9 : d0 + 3), hb)];
          }
          bias[nh] += q4.x * m4.x + q4.y * m4.y + q4.z * m4.z + q4.w * m4.w;
          const uint4 f = frag_hilo(q4.x * s4.x, q4.y * s4.y, q4.z * s4.z, q4.w * s4.w);
          frag[(nh * 8 + j) * 32 + lane] = (r & 1) ? make_uint2(f.y, f.w) : make_uint2(f.x, f.z);
        }
      }
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        bias[nh] += __shfl_xor_sync(0xffffffffu, bias[nh], 1);
        bias[nh] += __shfl_xor_sync(0xffffffffu, bias[nh], 2);
        if (c == 0 && (r & 1) == 0) bias_s[(4 * nh + (r >> 1)) * GW + gw] = bias[nh];
      }
    }
    // Outlier corrections of this warp's 64 tokens, in two parts: the fixed slots and the
    // page's widest channels, then the entries beyond the slots.
    const PageHeader* hdr = (const PageHeader*)(st + g.hdr_off);
    const bool spilled = cold && (hdr->flags & TQ_PAGE_SPILLED) != 0;
    auto fixed_corrections = [&]() {
      // Outlier corrections of this warp's 64 tokens (a lane owns tokens lane and lane + 32 of
      // the strip).  The page keeps the first TQ_ELL_SLOTS outliers of every token in fixed
      // slots, so the common case is a fixed number of independent, conflict-free rounds.
      constexpr int NI = TPW / 32;  // tokens of the strip per lane
      float cacc[NI][G];
#pragma unroll
      for (int i = 0; i < NI; ++i)
#pragma unroll
        for (int gg = 0; gg < G; ++gg) cacc[i][gg] = 0.0f;
      if (!spilled) {
        const uint16_t* ell_d = (const uint16_t*)(st + g.hdr_off + TQ_ELL_OFF) + TPW * gw + lane;
        const uint8_t* ell_c = st + g.hdr_off + TQ_ELL_COL_OFF + TPW * gw + lane;
#pragma unroll
        for (int j = 0; j < TQ_ELL_SLOTS; ++j) {
#pragma unroll
          for (int i = 0; i < NI; ++i) {
            const float delta = __half2float(__ushort_as_half(ell_d[j * 256 + 32 * i]));
            const float* qrow = qc + (int)ell_c[j * 256 + 32 * i] * QP;
            if (G >= 4) {
#pragma unroll
              for (int g4 = 0; g4 < G / 4; ++g4) {
                const float4 qv = *(const float4*)(qrow + (G == 8 ? g4 * (TQ_D * 4) : 4 * g4));
                cacc[i][4 * g4 + 0] += qv.x * delta;
                cacc[i][4 * g4 + 1] += qv.y * delta;
                cacc[i][4 * g4 + 2] += qv.z * delta;
                cacc[i][4 * g4 + 3] += qv.w * delta;
              }
            } else {
#pragma unroll
              for (int gg = 0; gg < G; ++gg) cacc[i][gg] += qrow[gg] * delta;
            }
          }
        }
      }
      // the widest channels of the page: their table rounding error, times a large
      // weight, would show in the scores, so it is added back here token by token
      {
        const uint16_t* side = (const uint16_t*)(st + g.hdr_off + TQ_SIDE_OFF) + TPW * gw;
        uint32_t sd[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) sd[i] = side[32 * i + lane];
#pragma unroll
        for (int j = 0; j < TQ_WIDE; ++j) {
          const int wch = hdr->wide[j];
          const float sc = scale[wch];
          const float* qrow = qc + q_row(wch) * QP;
          float dl[NI];
#pragma unroll
          for (int i = 0; i < NI; ++i) dl[i] = dtab[(sd[i] >> (4 * j)) & 15u] * sc;
          float qv[G];
          if (G >= 4) {
#pragma unroll
            for (int g4 = 0; g4 < G / 4; ++g4) {
              const float4 q4 = *(const float4*)(qrow + (G == 8 ? g4 * (TQ_D * 4) : 4 * g4));
              qv[4 * g4] = q4.x; qv[4 * g4 + 1] = q4.y; qv[4 * g4 + 2] = q4.z; qv[4 * g4 + 3] = q4.w;
            }
          } else {
#pragma unroll
            for (int gg = 0; gg < G; ++gg) qv[gg] = qrow[gg];
          }
#pragma unroll
          for (int gg = 0; gg < G; ++gg)
#pragma unroll
            for (int i = 0; i < NI; ++i) cacc[i][gg] += qv[gg] * dl[i];
        }
      }
#pragma unroll
      for (int i = 0; i < NI; ++i)
#pragma unroll
        for (int gg = 0; gg < G; ++gg) corr_w[gg * SM::CORR_STRIDE + 32 * i + lane] = cacc[i][gg];
    };
    auto overflow_corrections = [&]() {
      // Entries beyond the fixed slots (ordered by token), or, for a spilled page, the whole
      // list from the pool: a lane per entry, the entries of a token summed by the first lane
      // of their run (fixed order, so the result does not depend on timing), which adds the
      // sum to the strip.
      // (the page lists its overflow entries by 64-token quarter)
      const int s0 = spilled ? 0 : (int)hdr->ovf_start[(TPW * gw) >> 6];
      const int s1 = spilled ? (int)hdr->cnt : (int)hdr->ovf_start[((TPW * gw) >> 6) + 1];
      if (s1 > s0) {
        const uint32_t* list =
            spilled ? a.pool_dec + (unit0 + tl.u) * (size_t)g.pool_entries + hdr->off
                    : (const uint32_t*)(st + g.hdr_off + TQ_OVF_OFF);
        for (int eb = s0; eb < s1; eb += 32) {
          __syncwarp();
          const int e = eb + lane;
          const bool valid = e < s1;
          const uint32_t wv = valid ? list[e] : 0u;
          const int tok = valid ? (int)(wv >> 24) : -1 - lane;
          const bool mine = valid && tok / TPW == gw;
          const float delta =
              mine ? __half2float(__ushort_as_half((unsigned short)(wv & 0xffffu))) : 0.0f;
          const float* qrow = qc + q_row((wv >> 16) & 127) * QP;
          float pv[G];
          if (G >= 4) {
#pragma unroll
            for (int g4 = 0; g4 < G / 4; ++g4) {
              const float4 qv = *(const float4*)(qrow + (G == 8 ? g4 * (TQ_D * 4) : 4 * g4));
              pv[4 * g4] = qv.x * delta; pv[4 * g4 + 1] = qv.y * delta;
              pv[4 * g4 + 2] = qv.z * delta; pv[4 * g4 + 3] = qv.w * delta;
            }
          } else {
#pragma unroll
            for (int gg = 0; gg < G; ++gg) pv[gg] = qrow[gg] * delta;
          }
          // Entries of one token are neighbours (the list is ordered by token); the first lane
          // of each run adds up its run in lane order.  Runs are short (a token rarely has more
          // than two entries here), so this takes one or two rounds of shuffles.
          const int prev = __shfl_up_sync(0xffffffffu, tok, 1);
          const bool first = lane == 0 || prev != tok;
          const unsigned starts = __ballot_sync(0xffffffffu, first);
          const unsigned later = lane == 31 ? 0u : (starts >> (lane + 1)) << (lane + 1);
          const int run_end = later ? __ffs((int)later) - 1 : 32;  // first lane of the next run
          const int longest = __reduce_max_sync(0xffffffffu, first ? run_end - lane : 0);
          for (int o = 1; o < longest; ++o) {
#pragma unroll
            for (int gg = 0; gg < G; ++gg) {
              const float nv = __shfl_down_sync(0xffffffffu, pv[gg], o);
              if (first && lane + o < run_end) pv[gg] += nv;
            }
          }
          if (mine && first) {
#pragma unroll
            for (int gg = 0; gg < G; ++gg) corr_w[gg * SM::CORR_STRIDE + (tok & (TPW - 1))] += pv[gg];
          }
        }
        __syncwarp();
      }
    };
    if (cold) {
      fixed_corrections();
      overflow_corrections();
    }
    group_sync();  // fragments and bias of all four warps are in place
    if (warp == 0) TQ_TRACE(4);

    uint32_t breg[NH][8][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint2 f = frag[(nh * 8 + j) * 32 + lane];
        breg[nh][j][0] = f.x;
        breg[nh][j][1] = f.y;
      }

    if (cold) {
      float bias[NH];
      const float* corr[NH];
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        bias[nh] = 0.0f;
#pragma unroll
        for (int w4 = 0; w4 < GW / 4; ++w4) {
          const float4 b4 = *(const float4*)(bias_s + hc[nh] * GW + 4 * w4);
          bias[nh] += (b4.x + b4.y) + (b4.z + b4.w);
        }
        corr[nh] = corr_w + hc[nh] * SM::CORR_STRIDE + r;
      }
      const float* norms = (const float*)(st + g.norm_off);
      const uint8_t* vcodes = st + g.v_off;
      // Score tiles of 16 tokens (the lane looks up the codes of tokens r and r + 8; even and
      // odd k-steps accumulate separately: two independent chains per column group), and the
      // value tiles of 16 tokens.  The loop below is unrolled with the score phase of strip
      // h+1 placed before the value phase of strip h: the two are independent, so the
      // scheduler can fill the lookup and tensor-core latencies of one with the other.
      float C[NH][2][4];
      auto score_phase = [&](int half) {
        const int T0 = TPW * gw + 16 * half;
        uint32_t kw[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint4 kc = *(const uint4*)(st + (T0 + 8 * nt + r) * 64 + c * 16);
          kw[nt][0] = kc.x; kw[nt][1] = kc.y; kw[nt][2] = kc.z; kw[nt][3] = kc.w;
        }
#pragma unroll
        for (int nh = 0; nh < NH; ++nh)
#pragma unroll
          for (int x = 0; x < 2; ++x) C[nh][x][0] = C[nh][x][1] = C[nh][x][2] = C[nh][x][3] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t af[4];  // {token r | r+8} x {channels of rows 2c.. | 2c+8..}
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const uint32_t w = kw[nt][j >> 1];
            const uint32_t i0 = __byte_perm(w, 0, 0x4440 + 2 * (j & 1));
            const uint32_t i1 = __byte_perm(w, 0, 0x4441 + 2 * (j & 1));
            af[nt] = lut_ld(lutk + i0 * 128);
            af[2 + nt] = lut_ld(lutk + i1 * 128);
          }
#pragma unroll
          for (int nh = 0; nh < NH; ++nh) mma16816(C[nh][j & 1], af, breg[nh][j][0], breg[nh][j][1]);
        }
      };
      auto value_phase = [&](int half, uint32_t pb0, uint32_t pb1) {
        const int gq = HALVES * gw + half;
        if (VB == 4) {
          const uint8_t* gb = vcodes + gq * 1024 + lane * 16;
          const uint4 r0 = *(const uint4*)gb, r1 = *(const uint4*)(gb + 512);
          const uint32_t rec[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            const uint32_t w = rec[mt];  // pairs 4mt .. 4mt+3
            uint32_t af[4];
            af[0] = lut_ld(lutv + __byte_perm(w, 0, 0x4440) * 128);
            af[1] = lut_ld(lutv + __byte_perm(w, 0, 0x4442) * 128);
            af[2] = lut_ld(lutv + __byte_perm(w, 0, 0x4441) * 128);
            af[3] = lut_ld(lutv + __byte_perm(w, 0, 0x4443) * 128);
            mma16816(acc[mt], af, pb0, pb1);
          }
        } else {
          const uint8_t* gb = vcodes + gq * 768 + lane * 8;
          const uint2 r0 = *(const uint2*)gb, r1 = *(const uint2*)(gb + 256),
                      r2 = *(const uint2*)(gb + 512);
          const uint32_t rec[7] = {r0.x, r0.y, r1.x, r1.y, r2.x, r2.y, 0u};
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            uint32_t af[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // a0: pair 4mt, a1: pair 4mt+2, a2: pair 4mt+1, a3: pair 4mt+3; pair p is the
              // 6-bit field at bit 6p of the 192-bit record and must land at bits 7..12
              const int p = 4 * mt + ((e & 1) << 1) + (e >> 1);
              const int bit = 6 * p, wd = bit >> 5, sh = bit & 31;
              uint32_t f;
              if (sh < 7) f = rec[wd] << (7 - sh);
              else if (sh > 26) f = __funnelshift_r(rec[wd], rec[wd + 1], sh - 7);
              else f = rec[wd] >> (sh - 7);
              af[e] = lut_ld((f & 0x1f80u) | lutv);
            }
            mma16816(acc[mt], af, pb0, pb1);
          }
        }
      };
      {
        float sv[HALVES][NH][2];
#pragma unroll
        for (int half = 0; half < HALVES; ++half) {
          score_phase(half);
#pragma unroll
          for (int nh = 0; nh < NH; ++nh) {
            // columns 2c, 2c+1 of the tile: the hi and lo weight parts of the lane's head (heads
            // beyond the group carry zero weights: finite scores nobody reads)
            const float s0 = (C[nh][0][0] + C[nh][1][0]) + (C[nh][0][1] + C[nh][1][1]);
            const float s1 = (C[nh][0][2] + C[nh][1][2]) + (C[nh][0][3] + C[nh][1][3]);
            sv[half][nh][0] = s0 + (bias[nh] + corr[nh][16 * half]);
            sv[half][nh][1] = s1 + (bias[nh] + corr[nh][16 * half + 8]);
          }
        }
        softmax_many(sv);
#pragma unroll
        for (int half = 0; half < HALVES; ++half) {
          const int T0 = TPW * gw + 16 * half;
          uint32_t pb0, pb1;
          prob_frags(sv[half], norms[T0 + r], norms[T0 + r + 8], pb0, pb1);
          value_phase(half, pb0, pb1);
        }
      }
    } else if (gw < htt / 16 && a.use_tmap) {
      // ---- hot tile, swizzled 16-bit rows: 8x8 matrix loads straight into fragments --------
      const int hot_len = plan->hot_len[tl.u];
      const int T0 = 16 * gw;                   // first token of this warp inside the tile
      const int base_tok = tl.idx * htt + T0;   // ... inside the hot window
      // lanes 8m .. 8m+7 address the rows of matrix m: tokens T0 + 8 (m >> 1) + 0..7, 16-byte
      // chunk (m & 1) of the current channel pair; chunk ch of row tr lives in the 8 KB half
      // ch >> 3 at tr * 128 + ((ch & 7) ^ (tr & 7)) * 16
      const int tr = T0 + 8 * (lane >> 4) + (lane & 7), m1 = (lane >> 3) & 1, sw = lane & 7;
      const uint32_t ka = smem_addr(st) + tr * 128, va = ka + 16384;
      const bool bf = g.kv_dtype == TQ_BF16;
      float sv[NH][2];
      const bool ok[2] = {base_tok + r < hot_len, base_tok + r + 8 < hot_len};
      {
        float C[NH][2][4] = {};  // [column group][k-step parity]: independent chains
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t kb[4];  // key rows: {tokens 0-7: k lo, k hi, tokens 8-15: k lo, k hi}
          ldsm_x4(kb, ka + (j >> 2) * 8192 + (((2 * (j & 3) + m1) ^ sw) << 4));
          if (bf) {
#pragma unroll
            for (int i = 0; i < 4; ++i) kb[i] = bf16x2_to_h2(kb[i]);
          }
          const uint32_t af[4] = {kb[0], kb[2], kb[1], kb[3]};
#pragma unroll
          for (int nh = 0; nh < NH; ++nh) mma16816(C[nh][j & 1], af, breg[nh][j][0], breg[nh][j][1]);
        }
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
          sv[nh][0] = (C[nh][0][0] + C[nh][1][0]) + (C[nh][0][1] + C[nh][1][1]);
          sv[nh][1] = (C[nh][0][2] + C[nh][1][2]) + (C[nh][0][3] + C[nh][1][3]);
        }
      }
      softmax16(sv, ok);
      // tokens past the end of the window have probability 0 (their rows hold finite values:
      // the rings start zeroed and are only ever written with tokens)
      uint32_t pb0, pb1;
      prob_frags(sv, 1.0f, 1.0f, pb0, pb1);
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        // transposed loads: {tokens 0-7 | 8-15} x {channels 16mt + 0..7 | + 8..15} arrive as
        // {rows r, rows r+8} x {k 0-7, k 8-15} of the A fragment, in matrix order
        uint32_t af[4];
        ldsm_x4_trans(af, va + (mt >> 2) * 8192 + (((2 * (mt & 3) + m1) ^ sw) << 4));
        if (bf) {
#pragma unroll
          for (int i = 0; i < 4; ++i) af[i] = bf16x2_to_h2(af[i]);
        }
        mma16816(acc[mt], af, pb0, pb1);
      }
    } else if (gw < htt / 16) {
      // ---- hot tile, plain rows (float32 rings, or no tensor maps): loads + conversion -----
      const int hot_len = plan->hot_len[tl.u];
      const int T0 = 16 * gw;                   // first token of this warp inside the tile
      const int base_tok = tl.idx * htt + T0;   // ... inside the hot window
      const uint8_t* kbase = st;
      const uint8_t* vbase = st + htt * TQ_D * esz;
      float sv[NH][2];
      const bool ok[2] = {base_tok + r < hot_len, base_tok + r + 8 < hot_len};
      {
        uint32_t kw[2][16];  // tokens r and r + 8, channels 32c .. 32c+31 as fp16 pairs
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint8_t* row = kbase + ((T0 + 8 * nt + r) * TQ_D + 32 * c) * esz;
          if (esz == 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 v4 = *(const uint4*)(row + 16 * i);
              kw[nt][4 * i] = v4.x; kw[nt][4 * i + 1] = v4.y;
              kw[nt][4 * i + 2] = v4.z; kw[nt][4 * i + 3] = v4.w;
            }
            if (g.kv_dtype == TQ_BF16) {
#pragma unroll
              for (int i = 0; i < 16; ++i) kw[nt][i] = bf16x2_to_h2(kw[nt][i]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 v4 = *(const float4*)(row + 16 * i);
              kw[nt][2 * i] = pack_h2(v4.x, v4.y);
              kw[nt][2 * i + 1] = pack_h2(v4.z, v4.w);
            }
          }
        }
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
          float C[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t af[4] = {kw[0][2 * j], kw[1][2 * j], kw[0][2 * j + 1], kw[1][2 * j + 1]};
            mma16816(C, af, breg[nh][j][0], breg[nh][j][1]);
          }
          sv[nh][0] = C[0] + C[1];
          sv[nh][1] = C[2] + C[3];
        }
      }
      softmax16(sv, ok);
      uint32_t pb0, pb1;
      prob_frags(sv, 1.0f, 1.0f, pb0, pb1);
      // value rows of tokens 2c, 2c+1, 2c+8, 2c+9, channels 16r .. 16r+15, as fp16 pairs
      uint32_t vr[4][8];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int tloc = 2 * c + (q4 & 1) + 8 * (q4 >> 1);
        const bool valid = base_tok + tloc < hot_len;
        const uint8_t* row = vbase + ((T0 + tloc) * TQ_D + 16 * r) * esz;
        if (esz == 2) {
          const uint4 x0 = *(const uint4*)row, x1 = *(const uint4*)(row + 16);
          vr[q4][0] = x0.x; vr[q4][1] = x0.y; vr[q4][2] = x0.z; vr[q4][3] = x0.w;
          vr[q4][4] = x1.x; vr[q4][5] = x1.y; vr[q4][6] = x1.z; vr[q4][7] = x1.w;
          if (g.kv_dtype == TQ_BF16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) vr[q4][i] = bf16x2_to_h2(vr[q4][i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 v4 = *(const float4*)(row + 16 * i);
            vr[q4][2 * i] = pack_h2(v4.x, v4.y);
            vr[q4][2 * i + 1] = pack_h2(v4.z, v4.w);
          }
        }
        if (!valid) {
#pragma unroll
          for (int i = 0; i < 8; ++i) vr[q4][i] = 0u;
        }
      }
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        uint32_t af[4];
        af[0] = __byte_perm(vr[0][mt], vr[1][mt], 0x5410);  // channel 16r+2mt,   tokens 2c, 2c+1
        af[1] = __byte_perm(vr[0][mt], vr[1][mt], 0x7632);  // channel 16r+2mt+1
        af[2] = __byte_perm(vr[2][mt], vr[3][mt], 0x5410);  // tokens 2c+8, 2c+9
        af[3] = __byte_perm(vr[2][mt], vr[3][mt], 0x7632);
        mma16816(acc[mt], af, pb0, pb1);
      }
    }
    // every read of the stage is complete before the group's next barrier, after which the
    // stage is refilled
    asm volatile("" ::: "memory");
    __syncwarp();
    if (warp == 0) TQ_TRACE(7);
  }
  if (cur_u >= 0) flush(cur_u, cur_kind);
  // A group's last tile is among the last NG of the share, so no refill is owed here.  After
  // a timed-out wait copies may still be in flight: they are waited for (bounded) before the
  // CTA gives up its shared memory.
  // (a thread starts a copy only after the tile it started before that has been consumed, so
  // its latest one is the only one that can still be under way)
  if (*abort_flag && last_fired >= 0)
    waiter.drain(full0 + 8 * (last_fired % (2 * NSTAGE)), (last_fired / (2 * NSTAGE)) & 1);
}

// Combine for the tensor-core kernel: one CTA per (sequence, KV head) merges the partials of
// every CTA and consumer group that owned tiles of the unit, in the fixed order (CTA, cold
// before hot, group) and in rounds with a running maximum, un-rotates the cold part once
// (acc @ Pi) and writes the output or the (m, l, o) state.  Partial maxima are in the log2
// domain.  Built for short dependency chains: the candidate slots are tested in parallel and
// compacted in order, and a round's maxima, sums and accumulator rows are loaded together.
// A CTA merges GH of the unit's G query heads (blockIdx.y picks which): all of them where a
// layer has many units, one where it has few and the merge is on the critical path.
template <int G, int GH>
__global__ void __launch_bounds__(TQ_D) combine_mma_kernel(MmaArgs a) {
  constexpr int RP = GH >= 8 ? 8 : (GH >= 4 ? 16 : (GH >= 2 ? 32 : 64));  // partials per round
  const int g0 = blockIdx.y * GH;  // first head of this CTA
  const tq_geom& g = a.g;
  const int unit = blockIdx.x, e = threadIdx.x, lane = e & 31, wid = e >> 5;
  const int seq = (a.unit_base + unit) / g.n_kv_heads, head = (a.unit_base + unit) % g.n_kv_heads;
  __shared__ float cs[GH][TQ_D];
  __shared__ const float* s_ptr[TQ_D];  // partials of the current chunk of candidates
  __shared__ unsigned char s_cold[TQ_D];
  __shared__ int s_wcount[TQ_D / 32];
  __shared__ float s_m[RP][GH], s_l[RP][GH], s_wgt[RP][GH];
  __shared__ float s_M[GH], s_L[GH], s_scale[GH];
  // This kernel is launched while the attention kernel may still be running (programmatic
  // dependent launch): its column of the rotation matrix, which no kernel writes, is fetched
  // first; everything the attention kernel produces is read after the wait.
  float pcol[TQ_D];
#pragma unroll
  for (int d = 0; d < TQ_D; ++d) pcol[d] = a.tables->pi[d * TQ_D + e];
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the plan: all of it requested at once (one round trip to global memory), the shares then
  // searched in shared memory
  const int n_cta = a.plan_g[0];
  const int p0 = a.plan_g[2 + unit], p1 = a.plan_g[3 + unit];
  const int pc = p0 + a.plan_g[3 + a.n_units + unit];
  __shared__ int share[200];
  for (int i = e; i <= a.n_cta; i += TQ_D) share[i] = a.plan_g[3 + 2 * a.n_units + i];
  __syncthreads();
  const int NG = a.n_groups;
  // the CTAs whose shares meet the unit's tiles [p0, p1): i0 = the last one that starts at or
  // before p0, i1 = the last one that starts before p1
  int i0 = 0, i1 = -1;
  if (p1 > p0) {
    int lo_i = 0, hi_i = n_cta - 1;
    while (lo_i < hi_i) {
      const int mid = (lo_i + hi_i + 1) >> 1;
      if (share[mid] <= p0) lo_i = mid; else hi_i = mid - 1;
    }
    i0 = lo_i;
    hi_i = n_cta - 1;
    while (lo_i < hi_i) {
      const int mid = (lo_i + hi_i + 1) >> 1;
      if (share[mid] < p1) lo_i = mid; else hi_i = mid - 1;
    }
    i1 = lo_i;
  }
  if (e < GH) {
    s_M[e] = NEG_BIG;
    s_L[e] = 0.0f;
  }
  float C[GH], Hh[GH];
#pragma unroll
  for (int gg = 0; gg < GH; ++gg) C[gg] = Hh[gg] = 0.0f;
  // candidate t = ((cta - i0) * 2 + kind) * NG + group, tested 128 at a time
  const int n_cand = (i1 - i0 + 1) * 2 * NG;
  for (int base = 0; base < n_cand; base += TQ_D) {
    const int t = base + e;
    bool valid = false;
    const float* ptr = nullptr;
    int kind = 0;
    if (t < n_cand) {
      const int w = t % NG, ck = t / NG;
      kind = ck & 1;
      const int i = i0 + (ck >> 1);
      // tiles of this kind that CTA i holds for the unit: positions [ra, rb); the tile at
      // position p belongs to consumer group (p - lo) % NG
      const int lo = share[i], hi = share[i + 1];
      const int ra = kind == 0 ? max(lo, p0) : max(lo, pc);
      const int rb = kind == 0 ? min(hi, pc) : min(hi, p1);
      const int cnt = rb - ra;
      if (cnt > 0) {
        const int first = (ra - lo) % NG;
        valid = cnt >= NG || (w - first + NG) % NG < cnt;
      }
      ptr = a.partials +
            ((((size_t)unit + i) * 2 + kind) * NG + w) * (size_t)(G * TQ_PART_STRIDE);
    }
    __syncthreads();  // the previous chunk's list is no longer in use
    const unsigned ball = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) s_wcount[wid] = __popc(ball);
    __syncthreads();
    int off = __popc(ball & ((1u << lane) - 1u)), n_chunk = 0;
    for (int w2 = 0; w2 < TQ_D / 32; ++w2) {
      if (w2 < wid) off += s_wcount[w2];
      n_chunk += s_wcount[w2];
    }
    if (valid) {
      s_ptr[off] = ptr;
      s_cold[off] = (unsigned char)(kind == 0);
    }
    __syncthreads();
    for (int r0 = 0; r0 < n_chunk; r0 += RP) {
      const int nr = min(RP, n_chunk - r0);
      // this round's accumulator rows (all loads independent; rows past the end repeat the
      // last one and are ignored), maxima and sums
      float av[RP][GH];
#pragma unroll
      for (int j = 0; j < RP; ++j) {
        const float* pp = s_ptr[r0 + min(j, nr - 1)] + 2 + e;
#pragma unroll
        for (int gg = 0; gg < GH; ++gg) av[j][gg] = pp[(g0 + gg) * TQ_PART_STRIDE];
      }
      if (e < nr * GH) {
        const int j = e / GH, gg = e % GH;
        const float* pp = s_ptr[r0 + j] + (g0 + gg) * TQ_PART_STRIDE;
        s_m[j][gg] = pp[0];
        s_l[j][gg] = pp[1];
      }
      __syncthreads();
      // the round's maxima and sums: a warp per head, a lane per partial (two where a round
      // holds 64), reduced in a fixed tree, so the result does not depend on timing
      for (int gg = wid; gg < GH; gg += TQ_D / 32) {
        constexpr int PL = (RP + 31) / 32;  // partials per lane
        float mj[PL], lj[PL];
        float mx = s_M[gg];
#pragma unroll
        for (int k = 0; k < PL; ++k) {
          const int j = lane + 32 * k;
          const bool live = j < nr && j < RP;
          lj[k] = live ? s_l[j < RP ? j : 0][gg] : 0.0f;
          mj[k] = live ? s_m[j < RP ? j : 0][gg] : NEG_BIG;
          if (lj[k] > 0.0f) mx = fmaxf(mx, mj[k]);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float ls = 0.0f;
#pragma unroll
        for (int k = 0; k < PL; ++k) {
          const int j = lane + 32 * k;
          const float wgt = lj[k] > 0.0f ? exp2f(mj[k] - mx) : 0.0f;
          if (j < RP) s_wgt[j][gg] = wgt;
          ls += lj[k] * wgt;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
        const float old_m = s_M[gg], old_l = s_L[gg];
        __syncwarp();
        if (lane == 0) {
          const float sc = exp2f(old_m - mx);
          s_scale[gg] = sc;
          s_M[gg] = mx;
          s_L[gg] = old_l * sc + ls;
        }
      }
      __syncthreads();
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        C[gg] *= s_scale[gg];
        Hh[gg] *= s_scale[gg];
      }
#pragma unroll
      for (int j = 0; j < RP; ++j) {
        if (j < nr) {
          const bool cold = s_cold[r0 + j] != 0;
#pragma unroll
          for (int gg = 0; gg < GH; ++gg) {
            const float wgt = s_wgt[j][gg];
            const float v = wgt > 0.0f ? av[j][gg] * wgt : 0.0f;
            if (cold) C[gg] += v; else Hh[gg] += v;
          }
        }
      }
      __syncthreads();  // s_m / s_l / s_wgt are rewritten by the next round
    }
  }
#pragma unroll
  for (int gg = 0; gg < GH; ++gg) cs[gg][e] = C[gg];
  __syncthreads();
  float o[GH];
#pragma unroll
  for (int gg = 0; gg < GH; ++gg) o[gg] = 0.0f;
#pragma unroll
  for (int d = 0; d < TQ_D; ++d) {
#pragma unroll
    for (int gg = 0; gg < GH; ++gg) o[gg] += cs[gg][d] * pcol[d];
  }
  if (a.xchg_on) {
    // Publish this CTA's rows to every rank (peer stores), signal them, then wait for the same
    // rows of the other ranks and merge in rank order; the last CTA of the grid closes the
    // exchange.
    const XchgDev& x = a.xchg;
    const int row0 = seq * g.n_q_heads + head * G + g0;
    const unsigned ep = xchg_epoch(x);
    const int slot = (int)(ep & 1u);
    if (x.phases & 1) {
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) {
        const float val = o[gg] + Hh[gg];
        const float L = s_L[gg];
        const float m_nat = L > 0.0f ? s_M[gg] * 0.6931471805599453f : -INFINITY;
        for (int p = 0; p < x.world; ++p) {
          float* dst = xchg_row(x, p, slot, x.rank, row0 + gg);
          if (e == 0) {
            dst[0] = m_nat;
            dst[1] = L;
          }
          dst[2 + e] = val;
        }
      }
      __syncthreads();
#pragma unroll
      for (int gg = 0; gg < GH; ++gg) xchg_signal(x, e, slot, row0 + gg, ep);
    }
    if (x.phases & 2) {
      __shared__ int s_fail;
      if (e == 0) s_fail = 0;
      __syncthreads();
#pragma unroll
      for (int gg = 0; gg < GH; ++gg)
        if (!xchg_wait(x, e, slot, row0 + gg, ep)) s_fail = 1;
      __syncthreads();
      const bool fail = s_fail != 0;
#pragma unroll
      for (int gg = 0; gg < GH; ++gg)
        a.out[(size_t)(row0 + gg) * TQ_D + e] = fail ? 0.0f : xchg_merge_row(x, slot, row0 + gg, e);
      __syncthreads();
      if (e == 0) xchg_close(x, gridDim.x * gridDim.y, ep);
    }
    return;
  }
#pragma unroll
  for (int gg = 0; gg < GH; ++gg) {
    const size_t row = (size_t)seq * g.n_q_heads + head * G + g0 + gg;
    const float val = o[gg] + Hh[gg];
    const float L = s_L[gg];
    if (a.mlo != nullptr) {
      float* rr = a.mlo + row * TQ_PART_STRIDE;
      if (e == 0) {
        // natural-log domain, like the general kernel and tq_lse_combine
        rr[0] = L > 0.0f ? s_M[gg] * 0.6931471805599453f : -INFINITY;
        rr[1] = L;
      }
      rr[2 + e] = val;
    } else {
      a.out[row * TQ_D + e] = L > 0.0f ? val / L : 0.0f;
    }
  }
}

// Units of a layer one launch covers: the largest multiple of the KV head count that fits
// the shared-memory plan.  A layer with more units takes several launches, each with its own
// plan and partial slots in the scratch region.
int chunk_units(const tq_geom& g) { return MAX_UNITS / g.n_kv_heads * g.n_kv_heads; }
size_t chunk_bytes(const tq_geom& g, size_t units) {
  return TQ_MMA_PLAN_BYTES +
         align_up((units + 192) * 2 * MAX_NG * (size_t)g.group * TQ_PART_STRIDE * sizeof(float), 256);
}

template <int G, int VB>
int launch_t(MmaArgs a, cudaStream_t st, tq_ctx* ctx, bool first, bool last) {
  using CF = Cfg<G, VB>;
  using SM = typename CF::SM;
  static bool attr_set[16] = {};
  int dev = ctx->device;
  if (!attr_set[dev & 15]) {
    TQ_CUDA(cudaFuncSetAttribute(decode_mma_kernel<G, VB>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL));
    attr_set[dev & 15] = true;
  }
  // per-kernel timing brackets the attention kernel and the combine kernel of a one-launch
  // layer; with several launches the first bracket also holds the earlier launches' combines
  cudaEvent_t e0 = first ? tq_prof_event(ctx, 0) : nullptr;
  cudaEvent_t e1 = last ? tq_prof_event(ctx, 1) : nullptr;
  cudaEvent_t e2 = last ? tq_prof_event(ctx, 2) : nullptr;
  if (e0) cudaEventRecord(e0, st);
  a.n_groups = CF::NG;
  // Either kernel may be scheduled before its predecessor in the stream has finished (where
  // SMs are free) and waits for the predecessor's results itself (griddepcontrol.wait).
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3((unsigned)a.n_cta);
  cfg.blockDim = dim3(CF::THREADS);
  cfg.dynamicSmemBytes = SM::TOTAL;
  CUtensorMap tmk, tmv;
  std::memcpy(&tmk, ctx->tmap_hot[0], sizeof(CUtensorMap));
  std::memcpy(&tmv, ctx->tmap_hot[1], sizeof(CUtensorMap));
  TQ_CUDA(cudaLaunchKernelEx(&cfg, decode_mma_kernel<G, VB>, a, tmk, tmv));
  if (e1) cudaEventRecord(e1, st);
  cfg.blockDim = dim3(TQ_D);
  cfg.dynamicSmemBytes = 0;
  if (G > 1 && a.n_units <= 64) {  // few units: a CTA per query head, the merge is latency
    cfg.gridDim = dim3((unsigned)a.n_units, G);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, combine_mma_kernel<G, 1>, a));
  } else {
    cfg.gridDim = dim3((unsigned)a.n_units);
    TQ_CUDA(cudaLaunchKernelEx(&cfg, combine_mma_kernel<G, G>, a));
  }
  if (e2) {
    cudaEventRecord(e2, st);
    tq_prof_commit(ctx);
  }
  ctx->last_launches += 2;
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}

}  // namespace

// Builds the tensor maps of the two hot rings (16-bit element types only).  The driver
// function is looked up through the runtime, so the library does not link against libcuda.
static void build_hot_tensor_maps(tq_ctx* ctx) {
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  ctx->tmap_state = -1;
  const tq_geom& g = ctx->g;
  if (g.kv_dtype == TQ_F32) return;
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || fn == nullptr) {
    cudaGetLastError();
    return;
  }
  const cuuint64_t rows = (cuuint64_t)g.n_layers * g.n_seqs * g.n_kv_heads * g.hot_cap;
  const cuuint64_t dims[2] = {(cuuint64_t)TQ_D, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)TQ_D * 2};  // bytes between rows
  const cuuint32_t box[2] = {64, 64};                     // 64 channels (128 B) x 64 tokens
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt =
      g.kv_dtype == TQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  void* bases[2] = {ctx->b.hot_k, ctx->b.hot_v};
  for (int i = 0; i < 2; ++i) {
    CUtensorMap m;
    if (((encode_fn)fn)(&m, dt, 2, bases[i], dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return;
    std::memcpy(ctx->tmap_hot[i], &m, sizeof(m));
  }
  ctx->tmap_state = 1;
}

// Bytes of scratch the tensor-core path needs for `units` (sequence, KV head) pairs.
size_t tq_mma_scratch_bytes(const tq_geom& g, size_t units) {
  const size_t cu = (size_t)std::max(chunk_units(g), 1);
  size_t bytes = TQ_MMA_TRACE_BYTES;
  for (size_t u0 = 0; u0 < units; u0 += cu) bytes += chunk_bytes(g, std::min(cu, units - u0));
  return bytes;
}

int tq_launch_decode_mma(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                         int block_end, int with_hot, float* out, float* mlo, cudaStream_t st,
                         bool* handled, const tq_xchg* xchg, int xchg_phases) {
  const tq_geom& g = ctx->g;
  *handled = false;
  const int n_units = g.n_seqs * g.n_kv_heads;
  const int G = g.group;
  if (ctx->force_generic) return TQ_OK;
  if (g.key_mode == TQ_KEYS_POLAR) return TQ_OK;  // the legacy key format: general kernel
  if (g.block_tokens != BLK || (G != 1 && G != 2 && G != 4 && G != 8) ||
      g.n_kv_heads > MAX_UNITS || g.hot_cap % 64 != 0)
    return TQ_OK;
  int sm_count = 148;
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, ctx->device);
  MmaArgs a;
  a.g = g;
  a.pages = (const uint8_t*)ctx->b.pages;
  a.hot_k = (const uint8_t*)ctx->b.hot_k;
  a.hot_v = (const uint8_t*)ctx->b.hot_v;
  a.pool_dec = (const uint32_t*)ctx->b.pool_dec;
  a.seq_len = (const int32_t*)((const uint8_t*)ctx->b.state + state_len_off(g));
  a.tables = (const Tables*)ctx->b.tables;
  a.q = q;
  // scratch region: 4 KB of trace stamps, then per launch {8 KB plan for the combine, partials}
  a.trace = ctx->trace_on ? (unsigned long long*)ctx->b.scratch : nullptr;
  a.out = out;
  a.mlo = mlo;
  a.status = (int32_t*)((uint8_t*)ctx->b.state + state_status_off(g));
  a.layer = layer;
  a.q_dtype = q_dtype;
  a.n_cta = std::min(sm_count, 192);
  a.block_begin = block_begin;
  a.block_end = block_end;
  a.with_hot = with_hot;
  a.scale_log2 = 1.4426950408889634f / sqrtf((float)TQ_D);
  a.spin_limit = ctx->wait_limit > 0 ? ctx->wait_limit : SPIN_LIMIT;
  a.withhold_tile = ctx->withhold_tile;
  if (ctx->tmap_state == 0) build_hot_tensor_maps(ctx);
  a.use_tmap = ctx->tmap_state == 1 ? 1 : 0;
  a.xchg_on = 0;
  if (xchg != nullptr) {
    // (one launch must cover the layer: the exchange is closed by the last CTA of one grid)
    if (n_units > chunk_units(g) || xchg->rows != g.n_seqs * g.n_q_heads) return TQ_OK;
    TQ_REQUIRE(tq_xchg_view(xchg, xchg_phases, &a.xchg), TQ_ERR_INVALID,
               "a peer region is not connected");
    a.xchg_on = 1;
  }
  *handled = true;
  ctx->last_launches = 0;
  ctx->last_kernel = TQ_KERNEL_TENSOR_CORE;
  const int cu = chunk_units(g);
  uint8_t* region = (uint8_t*)ctx->b.scratch + TQ_MMA_TRACE_BYTES;
  for (int u0 = 0; u0 < n_units; u0 += cu) {
    a.unit_base = u0;
    a.n_units = std::min(cu, n_units - u0);
    a.plan_g = (int*)region;
    a.partials = (float*)(region + TQ_MMA_PLAN_BYTES);
    region += chunk_bytes(g, (size_t)a.n_units);
    const bool first = u0 == 0, last = u0 + cu >= n_units;
    int rc = TQ_ERR_UNSUPPORTED;
#define TQ_CASE(GG, VV) \
  if (G == GG && g.value_bits == VV) rc = launch_t<GG, VV>(a, st, ctx, first, last);
    TQ_CASE(1, 3) TQ_CASE(2, 3) TQ_CASE(4, 3) TQ_CASE(8, 3)
    TQ_CASE(1, 4) TQ_CASE(2, 4) TQ_CASE(4, 4) TQ_CASE(8, 4)
#undef TQ_CASE
    if (rc != TQ_OK) return rc;
  }
  return TQ_OK;
}
