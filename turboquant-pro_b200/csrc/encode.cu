// Append path: key encoder (per-channel asymmetric NF4 + fp16 outlier side-list), value
// encoder (PolarQuant: norm + rotated Lloyd-Max direction codes), hot-ring writer.
//
// Both encoders reproduce the reference's numpy arithmetic bit for bit, which pins the
// evaluation order: sequential float32 sums over tokens, the 8-accumulator norm, a
// multiply-then-add (never fused) rotation.  Every such operation uses the explicit
// round-to-nearest intrinsics (__fadd_rn, __fmul_rn, __fdiv_rn, __fsqrt_rn), which the
// compiler never contracts into FMAs.
#include "common.cuh"

namespace {

struct EncodeArgs {
  tq_geom g;
  uint8_t* pages;
  void* hot_k;
  void* hot_v;
  uint32_t* pool_dec;
  uint16_t* pool_val;
  PageMeta* page_meta;
  int32_t* seq_len;      // [L][B]
  uint32_t* pool_cursor; // [L][B][H]
  int32_t* status;
  const Tables* tables;
  const float* bias_means;  // given key zero-points [max_blocks][H][D], or null
  const void* k;
  const void* v;
  int layer, seq_begin, seq_count, n_tokens, max_new_blocks;
  int64_t seq_stride, tok_stride, head_stride;
  // PolarQuant keys (TQ_KEYS_POLAR): the value encoder also runs over the keys, writing their
  // codes where the per-channel codes would go and their norms over the scale / mean arrays
  int polar_keys_pass;
};

// Where token `pos` of (seq, head) currently lives: positions below n0 are already in the
// hot ring, the rest are in the caller's tensor.
template <int DT>
struct TokenSource {
  const void* ring;
  const void* in;
  int n0, cap;
  int64_t tok_stride;
  // one load from a selected address (no branch: loads of several positions can then be
  // in flight together)
  TQ_DEV float ld(int pos, int d) const {
    const bool old = pos < n0;
    const void* base = old ? ring : in;
    const size_t idx =
        old ? (size_t)(pos % cap) * TQ_D + d : (size_t)(pos - n0) * tok_stride + d;
    return Elem<DT>::ld(base, idx);
  }
};

template <int DT>
TQ_DEV TokenSource<DT> make_source(const EncodeArgs& a, const void* ring_base, const void* in_base,
                                   int seq, int head, int n0) {
  TokenSource<DT> s;
  s.ring = (const uint8_t*)ring_base +
           hot_offset_elems(a.g, a.layer, seq, head) * sizeof(typename Elem<DT>::type);
  s.in = (const uint8_t*)in_base +
         ((size_t)(seq - a.seq_begin) * a.seq_stride + (size_t)head * a.head_stride) *
             sizeof(typename Elem<DT>::type);
  s.n0 = n0;
  s.cap = a.g.hot_cap;
  s.tok_stride = a.tok_stride;
  return s;
}

// Packed minimum / maximum of two 16-bit floats (fp16 or bf16 by BF): the statistics of two
// tokens of a channel in one instruction.  The values are the tokens themselves, so nothing
// is rounded.
template <bool BF>
TQ_DEV uint32_t max2_16(uint32_t a, uint32_t b) {
  uint32_t r;
  if (BF) asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool BF>
TQ_DEV uint32_t min2_16(uint32_t a, uint32_t b) {
  uint32_t r;
  if (BF) asm("min.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("min.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool BF>
TQ_DEV float f16bits_to_float(uint32_t h) {
  return BF ? __uint_as_float(h << 16) : __half2float(__ushort_as_half((unsigned short)h));
}

// ---------------------------------------------------------------------------------------
// Key encoder.  One CTA per new cold block of one KV head, one thread per channel.
// Asymmetric NF4 (TQ_KEYS_NF4_ASYM):
//   mean   = (((x0 + x1) + x2) + ...) / S                      sequential float32 sum
//   scale  = max(max_s |x - mean|, 1e-8)
//   level  = fl(mean + fl(scale * NF4[l]));  code = first l minimising |fl(x - level_l)|
// Symmetric NF4 (TQ_KEYS_NF4): mean = 0, scale = max(max_s |x|, 1e-8), level = fl(scale * NF4[l]).
// Uniform (TQ_KEYS_UNIFORM): mean = min_s x, scale = fl(max(fl(max - min), 1e-8) / 15),
//   code = clip(round-half-even(fl(fl(x - min) / scale)), 0, 15).
// All modes: outliers are every token whose |x| reaches the channel's k-th largest magnitude.
// ---------------------------------------------------------------------------------------
// With STAGED the block's tokens are first brought into shared memory (every row with
// independent 16-byte loads, all in flight together) and the three passes read them from
// there; without it each pass reads global memory, one dependent load per token (kept for
// float32 tokens, whose block would take 128 KB).  A staged CTA runs two threads per channel
// (blockDim.x = 256): only the channel's sum has to visit the tokens in order, so the second
// thread takes the second half of the block in everything else and the two merge their
// running statistics once.
template <int DT, bool STAGED>
__global__ void __launch_bounds__(2 * TQ_D, 3) encode_keys_kernel(EncodeArgs a) {
  const tq_geom& g = a.g;
  const int seq = a.seq_begin + blockIdx.z;
  const int head = blockIdx.y;
  const int tid = threadIdx.x, d = tid & (TQ_D - 1), hf = tid >> 7, n_hf = blockDim.x >> 7;
  const int n0 = a.seq_len[a.layer * g.n_seqs + seq];
  const int nb0 = n_cold_blocks(n0, g.hot_window, g.block_tokens);
  const int nb1 = n_cold_blocks(n0 + a.n_tokens, g.hot_window, g.block_tokens);
  const int blk = nb0 + blockIdx.x;
  if (blk >= nb1) return;
  const int S = g.block_tokens;
  // this thread's tokens [t_lo, t_hi): the halves meet at an even token
  const int s_half = n_hf == 1 ? S : ((S / 2 + 1) & ~1);
  const int t_lo = min(hf * s_half, S), t_hi = hf == n_hf - 1 ? S : min((hf + 1) * s_half, S);
  const int pos0 = blk * S;
  const TokenSource<DT> src = make_source<DT>(a, a.hot_k, a.k, seq, head, n0);
  uint8_t* page = a.pages + page_offset(g, a.layer, seq, head, blk);
  const int kk = g.outlier_k;

  extern __shared__ __align__(16) uint8_t enck_rows[];  // [S][D] tokens of the block (STAGED)
  if (STAGED) {
    using T = typename Elem<DT>::type;
    constexpr int CH = TQ_D * (int)sizeof(T) / 16;  // 16-byte chunks per row
    const int n_chunks = S * CH;
#pragma unroll 8
    for (int i = tid; i < n_chunks; i += (int)blockDim.x) {
      const int t = i / CH, c = i % CH;
      const int pos = pos0 + t;
      const bool old = pos < n0;
      const T* row = old ? (const T*)src.ring + (size_t)(pos % src.cap) * TQ_D
                         : (const T*)src.in + (size_t)(pos - n0) * src.tok_stride;
      uint4 v;
      if (((uintptr_t)row & 15) == 0) {
        v = ((const uint4*)row)[c];
      } else {  // rows of an oddly strided caller tensor: element by element
        T tmp[16 / sizeof(T)];
#pragma unroll
        for (int e = 0; e < (int)(16 / sizeof(T)); ++e) tmp[e] = row[c * (16 / sizeof(T)) + e];
        v = *(const uint4*)tmp;
      }
      ((uint4*)enck_rows)[i] = v;
    }
  }
  // token t of this thread's channel
  auto ldx = [&](int t) -> float {
    return STAGED ? Elem<DT>::ld(enck_rows, (size_t)t * TQ_D + d) : src.ld(pos0 + t, d);
  };

  __shared__ int s_count;
  __shared__ uint32_t s_off;
  __shared__ int s_alloc;
  __shared__ int s_tok_cnt[256];    // outliers per token
  __shared__ unsigned char s_cnt_w[256][TQ_D / 32];  // ... of which on the channels of warp w
  __shared__ unsigned short s_row[258];   // start of every token's outliers in the side-list
  __shared__ unsigned short s_orow[258];  // start of every token's entries in the page's overflow list
  __shared__ int s_warp_sum[TQ_D / 32];
  // The level grid, and for 64 equal bins of [-1, 1] the grid cell (nearest level) that holds
  // the bin's left edge, a little to the left of it: pass 3 finds a token's two candidate
  // levels with it.  Usable when the cell borders lie further apart than a bin is wide.
  __shared__ float s_grid[16];
  __shared__ unsigned char s_bin[64];
  constexpr float BIN_EPS = 1.0e-4f;
  if (tid == 0) s_count = 0;
  if (tid < 16) s_grid[tid] = a.tables->grid[tid];
  __shared__ float s_scale[TQ_D];       // channel scales, to rank the widest channels
  __shared__ unsigned int s_side[256];  // per token: the codes of the four widest channels
  __shared__ float s_stat[10][TQ_D];  // running statistics on their way between the two halves
  // Once the halves have merged, the same words hold the block's outliers as pass 3 meets them
  // (token | channel << 8 | outlier channels below it in its warp << 16 | code << 24); they are
  // worked off afterwards, one per thread, instead of by one or two lanes of a warp at a time.
  uint32_t* s_list = (uint32_t*)&s_stat[0][0];
  constexpr int LIST_CAP = 10 * TQ_D;
  __shared__ int s_n_list;
  __shared__ float s_mu[TQ_D];
  if (tid == 0) s_n_list = 0;
  if (hf == 0) {
    s_side[d] = 0u;
    s_side[d + TQ_D] = 0u;
  }
  __syncthreads();
  bool grid_regular = true;  // ascending, cell borders at least 1.5 bins apart
  {
    float prev_mid = -2.0f;
#pragma unroll
    for (int l = 0; l < 15; ++l) {
      const float mid = 0.5f * (s_grid[l] + s_grid[l + 1]);
      grid_regular = grid_regular && s_grid[l] < s_grid[l + 1] && mid - prev_mid > 1.5f / 32.0f;
      prev_mid = mid;
    }
    grid_regular = grid_regular && s_grid[0] >= -1.0f && s_grid[15] <= 1.0f;
    if (tid < 64) {
      const float left = -1.0f + (float)tid * (1.0f / 32.0f) - BIN_EPS;
      int cell = 0;
#pragma unroll
      for (int l = 0; l < 15; ++l) cell += (0.5f * (s_grid[l] + s_grid[l + 1]) < left) ? 1 : 0;
      s_bin[tid] = (unsigned char)cell;
    }
  }

  // pass 1: sequential sum and the k largest magnitudes.  Up to eight of them (the usual
  // case: k = 5 at 256-token blocks) are kept in an ascending register array updated without
  // branches, t[j] <- min(max(|x|, t[j]), t[j+1]); larger k takes the insertion loop.
  constexpr int TK = 8;
  const bool small_k = kk <= TK;  // uniform over the grid
  float t8[TK];
#pragma unroll
  for (int i = 0; i < TK; ++i) t8[i] = -1.0f;
  float top[TQ_MAX_K_OUT];  // ascending; top[0] is the k-th largest (k > 8 only)
#pragma unroll
  for (int i = 0; i < TQ_MAX_K_OUT; ++i) top[i] = -1.0f;
  const int mode = g.key_mode;
  // (the first thread of a channel also carries the sum, over all tokens in order; more than
  // eight outliers per channel are tracked by that thread alone, over all tokens)
  // The first thread visits every token for the sum, so it takes the smaller share of the
  // other statistics: the shares are cut where the two threads' instruction counts meet.
  float acc = 0.0f, xmin = INFINITY, xmax = -INFINITY;
  const bool k5 = kk <= 5;  // uniform: the five largest suffice, kept in t8[3..7]
  // Staged 16-bit tokens are taken two at a time with packed instructions (even tokens in the
  // low halves, odd ones in the high halves: two top lists, merged at the end).
  constexpr bool PACKED = STAGED && DT != TQ_F32;
  const bool packed = PACKED && small_k && (S & 1) == 0;  // uniform
  const int own_cut = (n_hf == 1 || !small_k) ? S
                      : packed ? ((S * (k5 ? 96 : 108)) >> 8) & ~1
                               : ((S * (k5 ? 88 : 101)) >> 8) & ~1;
  int p1_lo = hf == 0 ? 0 : (small_k ? own_cut : t_lo);
  if (PACKED && packed) {
    constexpr bool BF = DT == TQ_BF16;
    constexpr uint32_t NEG1 = BF ? 0xBF80BF80u : 0xBC00BC00u;     // (-1, -1)
    constexpr uint32_t PINF = BF ? 0x7F807F80u : 0x7C007C00u, NINF = PINF | 0x80008000u;
    const unsigned short* rows16 = (const unsigned short*)enck_rows;
    uint32_t h8[TK], mn = PINF, mx = NINF;
#pragma unroll
    for (int i = 0; i < TK; ++i) h8[i] = NEG1;
    const int o_lo = hf == 0 ? 0 : own_cut, o_hi = hf == 0 ? own_cut : S;
    for (int t = o_lo; t < o_hi; t += 2) {
      const uint32_t b0 = rows16[(size_t)t * TQ_D + d], b1 = rows16[(size_t)(t + 1) * TQ_D + d];
      if (hf == 0) {
        const float x0 = f16bits_to_float<BF>(b0), x1 = f16bits_to_float<BF>(b1);
        acc = t == 0 ? x0 : __fadd_rn(acc, x0);
        acc = __fadd_rn(acc, x1);
      }
      const uint32_t xx = b0 | (b1 << 16), ax = xx & 0x7FFF7FFFu;
      mn = min2_16<BF>(mn, xx);
      mx = max2_16<BF>(mx, xx);
      if (!k5) {
#pragma unroll
        for (int j = 0; j < 3; ++j) h8[j] = min2_16<BF>(max2_16<BF>(ax, h8[j]), h8[j + 1]);
      }
#pragma unroll
      for (int j = 3; j < TK - 1; ++j) h8[j] = min2_16<BF>(max2_16<BF>(ax, h8[j]), h8[j + 1]);
      h8[TK - 1] = max2_16<BF>(ax, h8[TK - 1]);
    }
    // the even tokens' list, then the odd tokens' largest inserted one by one
#pragma unroll
    for (int j = 0; j < TK; ++j) t8[j] = f16bits_to_float<BF>(h8[j] & 0xFFFFu);
#pragma unroll
    for (int i = 0; i < TK; ++i) {
      const float ax = f16bits_to_float<BF>(h8[i] >> 16);
#pragma unroll
      for (int j = 0; j < TK - 1; ++j) t8[j] = fminf(fmaxf(ax, t8[j]), t8[j + 1]);
      t8[TK - 1] = fmaxf(ax, t8[TK - 1]);
    }
    xmin = fminf(f16bits_to_float<BF>(mn & 0xFFFFu), f16bits_to_float<BF>(mn >> 16));
    xmax = fmaxf(f16bits_to_float<BF>(mx & 0xFFFFu), f16bits_to_float<BF>(mx >> 16));
    p1_lo = hf == 0 ? own_cut : S;  // what is left for the loop below: the rest of the sum
  }
  for (int t = p1_lo; t < S; ++t) {
    const float x = ldx(t);
    if (hf == 0) acc = t == 0 ? x : __fadd_rn(acc, x);
    const bool own = (hf != 0 || t < own_cut) && !packed;
    const float ax = fabsf(x);
    if (own) {
      xmin = fminf(xmin, x);
      xmax = fmaxf(xmax, x);
    }
    if (small_k) {
      if (own) {
        if (!k5) {
#pragma unroll
          for (int j = 0; j < 3; ++j) t8[j] = fminf(fmaxf(ax, t8[j]), t8[j + 1]);
        }
#pragma unroll
        for (int j = 3; j < TK - 1; ++j) t8[j] = fminf(fmaxf(ax, t8[j]), t8[j + 1]);
        t8[TK - 1] = fmaxf(ax, t8[TK - 1]);
      }
    } else if (hf == 0 && ax > top[0]) {
      int i = 0;
      while (i + 1 < kk && top[i + 1] < ax) { top[i] = top[i + 1]; ++i; }
      top[i] = ax;
    }
  }
  if (n_hf > 1) {
    // Both threads of a channel end up with the statistics of the whole block: the second
    // hands over its eight largest and its extremes, the first merges them into its own and
    // hands the result back together with the sum (and the k-th largest when k > 8); the sum
    // and that value travel in the token-count array, which is not in use yet.
    float* s_sum = (float*)s_tok_cnt;
    if (hf == 1) {
#pragma unroll
      for (int j = 0; j < TK; ++j) s_stat[j][d] = t8[j];
      s_stat[8][d] = xmin;
      s_stat[9][d] = xmax;
    }
    __syncthreads();
    if (hf == 0) {
      xmin = fminf(xmin, s_stat[8][d]);
      xmax = fmaxf(xmax, s_stat[9][d]);
#pragma unroll
      for (int i = 0; i < TK; ++i) {  // the other half's eight largest, inserted one by one
        const float ax = s_stat[i][d];
#pragma unroll
        for (int j = 0; j < TK - 1; ++j) t8[j] = fminf(fmaxf(ax, t8[j]), t8[j + 1]);
        t8[TK - 1] = fmaxf(ax, t8[TK - 1]);
      }
#pragma unroll
      for (int j = 0; j < TK; ++j) s_stat[j][d] = t8[j];
      s_stat[8][d] = xmin;
      s_stat[9][d] = xmax;
      s_sum[d] = acc;
      s_sum[TQ_D + d] = top[0];
    }
    __syncthreads();
    if (hf == 1) {
#pragma unroll
      for (int j = 0; j < TK; ++j) t8[j] = s_stat[j][d];
      xmin = s_stat[8][d];
      xmax = s_stat[9][d];
      acc = s_sum[d];
      top[0] = s_sum[TQ_D + d];
    }
  }
  float kth_small = -1.0f;  // the k-th largest = element TK - k of the ascending eight
#pragma unroll
  for (int j = 0; j < TK; ++j) kth_small = (j == TK - kk) ? t8[j] : kth_small;
  // (the "sparse" zero-point keeps the mean on the masked channels only)
  const float mu = mode == TQ_KEYS_NF4_ASYM
                       ? (a.bias_means != nullptr
                              ? a.bias_means[((size_t)blk * g.n_kv_heads + head) * TQ_D + d]
                          : a.tables->mean_mask[d] ? __fdiv_rn(acc, (float)S)
                                                   : 0.0f)
                   : mode == TQ_KEYS_NF4 ? 0.0f
                                         : xmin;
  const float kth = (kk >= S || kk == 0) ? -1.0f : (small_k ? kth_small : top[0]);

  // The scale max_s |fl(x_s - mu)| is reached at the smallest or the largest token (rounding is
  // monotone), so it needs no pass of its own.
  float amax = mode == TQ_KEYS_NF4_ASYM
                   ? fmaxf(fabsf(__fsub_rn(xmax, mu)), fabsf(__fsub_rn(xmin, mu)))
                   : fmaxf(fabsf(xmax), fabsf(xmin));
  // pass 2: how many outliers this channel keeps, and which tokens they fall on
  int my_out = 0;
  for (int t = t_lo; t < t_hi; ++t) {
    float x = ldx(t);
    const bool is_out = kk > 0 && fabsf(x) >= kth;
    my_out += is_out ? 1 : 0;
    // (the loop is uniform over the warp: every lane takes part in the vote)
    const unsigned vote = __ballot_sync(0xffffffffu, is_out);
    if ((d & 31) == 0) s_cnt_w[t][d >> 5] = (unsigned char)__popc(vote);
  }
  amax = fmaxf(amax, 1e-8f);
  if (mode == TQ_KEYS_UNIFORM) amax = __fdiv_rn(fmaxf(__fsub_rn(xmax, xmin), 1e-8f), 15.0f);
  // from here on `amax` is the channel's scale in every mode: dense = mean + scale * grid[code]
  float lev[16];
#pragma unroll
  for (int l = 0; l < 16; ++l) {
    const float sl = __fmul_rn(amax, a.tables->grid[l]);
    lev[l] = mode == TQ_KEYS_NF4 ? sl : __fadd_rn(mu, sl);
  }

  if (hf == 0) {
    ((float*)(page + g.scale_off))[d] = amax;
    ((float*)(page + g.mean_off))[d] = mu;
    s_scale[d] = amax;
    s_mu[d] = mu;
  }
  // allocate this page's slice of the (layer, seq, head) outlier slab
  __syncthreads();
  // Rank of this channel by scale (0 = widest; ties go to the lower channel).  The codes of
  // the four widest channels are stored a second time, token by token, so that the decode
  // kernel can add their contribution at full float32 table precision: w * NF4 of such a
  // channel is large enough for the fp16 rounding of the table to show in the scores.
  int rank = 0;
  for (int o = 0; o < TQ_D; ++o) {
    const float so = s_scale[o];
    rank += (so > amax || (so == amax && o < d)) ? 1 : 0;
  }
  PageHeader* hdr = (PageHeader*)(page + g.hdr_off);
  if (rank < TQ_WIDE && hf == 0) hdr->wide[rank] = (uint8_t)d;
  if (kk > 0) atomicAdd(&s_count, my_out);
  __syncthreads();
  if (hf == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int t = 2 * d + i;
      int n = 0;
#pragma unroll
      for (int w = 0; w < TQ_D / 32; ++w) n += t < S ? (int)s_cnt_w[t][w] : 0;
      s_tok_cnt[t] = n;
    }
  }
  if (tid == 0) {
    int n = s_count;
    uint32_t off = 0;
    int alloc = 0;
    if (n > 0) {
      int n4 = (n + 3) & ~3;
      off = atomicAdd(&a.pool_cursor[unit_index(g, a.layer, seq, head)], (uint32_t)n4);
      if (off >= (uint32_t)g.pool_entries) {
        alloc = 0;
        off = 0;
      } else {
        alloc = min(n4, g.pool_entries - (int)off);
      }
      if (alloc < n4) atomicOr(a.status, TQ_STATUS_POOL_OVERFLOW);
    }
    s_off = off;
    s_alloc = alloc;
    PageMeta pm;
    pm.off = off;
    pm.cnt = (uint32_t)min(n, alloc);
    a.page_meta[unit_index(g, a.layer, seq, head) * g.max_blocks + blk] = pm;
    hdr->off = pm.off;  // the page carries its own copy for the decode kernel
    hdr->cnt = pm.cnt;
  }
  uint16_t* ell_delta = (uint16_t*)(page + g.hdr_off + TQ_ELL_OFF);  // [slot][token]
  uint8_t* ell_col = page + g.hdr_off + TQ_ELL_COL_OFF;               // [slot][token]
  uint32_t* ovf = (uint32_t*)(page + g.hdr_off + TQ_OVF_OFF);
  // exclusive prefix sums over tokens of the outlier counts and of the counts beyond the
  // fixed slots (both in one word: each total stays below 65536); the first thread of channel
  // d owns tokens 2d and 2d+1
  int c0 = 0, c1 = 0, o0 = 0;
  uint32_t mine = 0u, v = 0u;
  if (hf == 0) {
    c0 = s_tok_cnt[2 * d];
    c1 = s_tok_cnt[2 * d + 1];
    o0 = max(c0 - TQ_ELL_SLOTS, 0);
    const int o1 = max(c1 - TQ_ELL_SLOTS, 0);
    mine = (uint32_t)(c0 + c1) | ((uint32_t)(o0 + o1) << 16);
    v = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t nv = __shfl_up_sync(0xffffffffu, v, o);
      if ((d & 31) >= o) v += nv;
    }
    if ((d & 31) == 31) s_warp_sum[d >> 5] = (int)v;
  }
  __syncthreads();
  if (hf == 0) {
    uint32_t base = 0;
    for (int w = 0; w < (d >> 5); ++w) base += (uint32_t)s_warp_sum[w];
    const uint32_t excl = base + v - mine;
    s_row[2 * d] = (unsigned short)(excl & 0xffffu);
    s_row[2 * d + 1] = (unsigned short)((excl & 0xffffu) + c0);
    s_orow[2 * d] = (unsigned short)(excl >> 16);
    s_orow[2 * d + 1] = (unsigned short)((excl >> 16) + o0);
    if (d == TQ_D - 1) {
      s_row[256] = (unsigned short)((base + v) & 0xffffu);
      s_orow[256] = (unsigned short)((base + v) >> 16);
    }
    // slots the tokens do not use hold a zero delta on channel 0
    for (int j = c0; j < TQ_ELL_SLOTS; ++j) {
      ell_delta[j * 256 + 2 * d] = 0;
      ell_col[j * 256 + 2 * d] = 0;
    }
    for (int j = c1; j < TQ_ELL_SLOTS; ++j) {
      ell_delta[j * 256 + 2 * d + 1] = 0;
      ell_col[j * 256 + 2 * d + 1] = 0;
    }
  }
  __syncthreads();
  if (tid < 5) hdr->ovf_start[tid] = (uint16_t)min((int)s_orow[64 * tid], TQ_OVF_CAP);
  if (tid == 5) {
    // the in-page copy is complete unless the overflow list is too long or the pool slab
    // could not take every entry (then the pool's shorter list is the cache's content)
    const int n_ovf = (int)s_orow[256];
    hdr->ovf_n = (uint16_t)min(n_ovf, TQ_OVF_CAP);
    hdr->flags = (n_ovf > TQ_OVF_CAP || s_alloc < s_count) ? TQ_PAGE_SPILLED : 0;
  }
  __syncthreads();
  const size_t slab = unit_index(g, a.layer, seq, head) * (size_t)g.pool_entries + s_off;
  const int alloc = s_alloc;

  // pass 3: codes and outlier entries.  The nearest level of a token is found by a
  // tournament over the 16 distances in which the lower index wins a tie at every round (the
  // first minimum, like a strict-less scan from level 0, in four dependent steps instead of
  // fifteen), and two tokens are worked on together so that their chains overlap.
  // Where the levels of a channel are well separated (the scale is not tiny against the
  // mean, so that rounding cannot merge or reorder them) only two levels can be the nearest:
  // those of the one or two grid cells that meet the token's bin.  Every other level is
  // further away by at least BIN_EPS of the scale, far more than the rounding of a
  // difference, so comparing those two the way the reference does (rounded differences, the
  // lower index on a tie) gives the reference's first minimum.
  const float mu_eff = mode == TQ_KEYS_NF4 ? 0.0f : mu;
  const bool two_cand = grid_regular && mode != TQ_KEYS_UNIFORM && amax >= fabsf(mu_eff) * (1.0f / 512.0f);
  const float inv32 = 32.0f / amax;
  auto level_of = [&](int l) -> float {
    const float sl = __fmul_rn(amax, s_grid[l]);
    return mode == TQ_KEYS_NF4 ? sl : __fadd_rn(mu, sl);
  };
  auto nearest = [&](float x) -> int {
    if (mode == TQ_KEYS_UNIFORM) {
      const float qv = rintf(__fdiv_rn(__fsub_rn(x, mu), amax));  // ties to even, like np.round
      return (int)fminf(fmaxf(qv, 0.0f), 15.0f);
    }
    if (two_cand) {
      const int bin = min(max(__float2int_rd(fmaf(x - mu_eff, inv32, 32.0f)), 0), 63);
      const int i0 = s_bin[bin], i1 = min(i0 + 1, 15);
      const float d0 = fabsf(__fsub_rn(x, level_of(i0))), d1 = fabsf(__fsub_rn(x, level_of(i1)));
      return d1 < d0 ? i1 : i0;
    }
    float dv[16];
#pragma unroll
    for (int l = 0; l < 16; ++l) dv[l] = fabsf(__fsub_rn(x, lev[l]));
    int ix[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool up = dv[2 * j + 1] < dv[2 * j];
      dv[j] = up ? dv[2 * j + 1] : dv[2 * j];
      ix[j] = 2 * j + (up ? 1 : 0);
    }
#pragma unroll
    for (int w = 4; w >= 1; w >>= 1) {
#pragma unroll
      for (int j = 0; j < w; ++j) {
        const bool up = dv[2 * j + 1] < dv[2 * j];
        dv[j] = up ? dv[2 * j + 1] : dv[2 * j];
        ix[j] = up ? ix[2 * j + 1] : ix[2 * j];
      }
    }
    return ix[0];
  };
  // Stores outlier (token t, channel dch, value x, code `code`).  A token's outliers are stored
  // in channel order (the order of the reference's flat indices), so the side-list, and with it
  // every bit the decoder computes, is a function of the tokens alone: the entry's place is the
  // count of outlier channels below it (`bw` of them in its own group of 32 channels).
  auto put_outlier = [&](int t, int dch, int bw, int code, float x) {
    int below = bw;
    for (int w = 0; w < (dch >> 5); ++w) below += (int)s_cnt_w[t][w];
    const int slot = (int)s_row[t] + below;
    const __half hv = __float2half_rn(x);
    // the decoder's value of this position
    const float sl = __fmul_rn(s_scale[dch], s_grid[code]);
    const float dense = mode == TQ_KEYS_NF4 ? sl : __fadd_rn(s_mu[dch], sl);
    const __half delta = __float2half_rn(__fsub_rn(__half2float(hv), dense));
    const uint32_t ent = (uint32_t)__half_as_ushort(delta) | ((uint32_t)dch << 16) |
                         ((uint32_t)t << 24);
    if (slot < alloc) {
      a.pool_dec[slab + slot] = ent;
      a.pool_val[slab + slot] = __half_as_ushort(hv);
    }
    if (below < TQ_ELL_SLOTS) {
      ell_delta[below * 256 + t] = __half_as_ushort(delta);
      ell_col[below * 256 + t] = (uint8_t)q_row(dch);
    } else {
      const int oi = (int)s_orow[t] + below - TQ_ELL_SLOTS;
      if (oi < TQ_OVF_CAP) ovf[oi] = ent;
    }
  };
  for (int t0 = t_lo; t0 < t_hi; t0 += 2) {
    const float xa = ldx(t0), xb = ldx(min(t0 + 1, S - 1));
    const int best_a = nearest(xa), best_b = nearest(xb);
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
      const int t = t0 + sub;
      if (t >= t_hi) break;  // uniform over the warp
      const float x = sub ? xb : xa;
      const int best = sub ? best_b : best_a;
      if (rank < 4) atomicOr(&s_side[t], (unsigned int)best << (4 * rank));
      int other = __shfl_down_sync(0xffffffffu, best, 1);
      if ((d & 1) == 0) page[t * (TQ_D / 2) + (d >> 1)] = (uint8_t)(best | (other << 4));
      // A token's outliers are stored in channel order (the order of the reference's flat
      // indices), so the side-list, and with it every bit the decoder computes, is a function
      // of the tokens alone: this channel's place is the count of outlier channels below it.
      const bool is_out = kk > 0 && fabsf(x) >= kth;
      const unsigned vote = __ballot_sync(0xffffffffu, is_out);
      if (is_out) {
        const int bw = __popc(vote & ((1u << (d & 31)) - 1u));
        const int li = atomicAdd(&s_n_list, 1);
        if (li < LIST_CAP) {
          s_list[li] = (uint32_t)t | ((uint32_t)d << 8) | ((uint32_t)bw << 16) | ((uint32_t)best << 24);
        } else {  // (a block with more outliers than the list holds: in place)
          put_outlier(t, d, bw, best, x);
        }
      }
    }
  }
  __syncthreads();
  {
    const int n_list = min(s_n_list, LIST_CAP);
    for (int li = tid; li < n_list; li += (int)blockDim.x) {
      const uint32_t ent = s_list[li];
      const int t = (int)(ent & 255u), dch = (int)((ent >> 8) & 127u);
      const float x = STAGED ? Elem<DT>::ld(enck_rows, (size_t)t * TQ_D + dch) : src.ld(pos0 + t, dch);
      put_outlier(t, dch, (int)((ent >> 16) & 31u), (int)(ent >> 24), x);
    }
  }
  __syncthreads();
  if (hf == 0) {
    uint16_t* side = (uint16_t*)(page + g.hdr_off + TQ_SIDE_OFF);
    side[2 * d] = (uint16_t)s_side[2 * d];
    side[2 * d + 1] = (uint16_t)s_side[2 * d + 1];
    // padded token rows (block_tokens not a multiple of 16) keep code 0
    for (int t = S; t < g.block_tokens_pad; ++t)
      if ((d & 1) == 0) page[t * (TQ_D / 2) + (d >> 1)] = 0;
  }
}

// ---------------------------------------------------------------------------------------
// Rotation of the value encoder on tensor cores.  The reference's result is the unfused
// sequential float32 sum y_ch = ((u0*P0 + u1*P1) + u2*P2) + ... with every product and sum
// rounded separately; it lies within 127 * 2^-24 + 2^-24 < 7.7e-6 of the exact dot product
// (the absolute values of the 128 terms add up to at most |u| |column| <= 1).  The tensor-core
// form splits every operand into two fp16 parts, x = hi + lo * 2^-11 with hi = fp16(x) and
// lo = fp16((x - hi) * 2^11) (what is left is below 2^-24 |x|), and sums hi*hi into one
// float32 accumulator and hi*lo + lo*hi into another; the products are exact in float32, the
// dropped lo*lo term is below 2^-24 of a term, and the accumulators add eight (sixteen)
// 16-term tiles; the unit vector it rotates is x * (1 / norm), within 2^-22 of x / norm.
// That result lies within a few 1e-6 of the exact dot product, so the two
// differ by less than 1.6e-5; ROT_SLACK leaves a factor 2.5 on top of that.  A coordinate
// with a quantisation boundary inside the slack is computed again in the reference's order.
constexpr float ROT_SLACK = 4.0e-5f;
// Row stride (floats) of the token rows: the 8-threads-per-token phases (norms, unit vectors)
// then touch 32 different banks; and (halves) of the fp16 unit-vector rows: eight rows of an
// 8x8 matrix load then fall into eight different 16-byte bank groups.
constexpr int ENCV_XS = TQ_D + 8, ENCV_UH = TQ_D + 8;

TQ_DEV void enc_mma16816(float* c, const uint4& a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
TQ_DEV void enc_ldsm_x4(uint32_t* v, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(addr));
}
// x = hi + lo * 2^-11, both fp16
TQ_DEV void split_h(float x, __half& hi, __half& lo) {
  hi = __float2half_rn(x);
  lo = __float2half_rn((x - __half2float(hi)) * 2048.0f);
}
TQ_DEV uint32_t h2_bits(__half lo, __half hi) {
  return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

// ---------------------------------------------------------------------------------------
// Value encoder.  Persistent CTAs of two 128-thread halves that share one copy of the
// rotation matrix in shared memory (as ready-made tensor-core fragments); each half works on
// its own 16-token group of a new cold block.
//   norm = sqrt(pairwise sum of fl(x*x))      (numpy's 8-accumulator order for n = 128)
//   u    = x / max(norm, 1e-30)
//   y_ch = sequential, unfused sum over d of u_d * Pi[ch][d]
//   code = #{ j : boundary_j < y_ch }
// The rotation runs as Y^T = Pi . U^T on m16n8k16 tiles (rows: 16 channels, columns: 8
// tokens): warp w of the half owns channels 32w .. 32w+31, and lane (r, c) ends up with
// channels 16mt + r, 16mt + r + 8 and tokens 2c, 2c+1, 2c+8, 2c+9 - exactly the codes of
// its own lane record of the page's value layout, which it packs and stores itself.
// ---------------------------------------------------------------------------------------
constexpr int ENCV_HALVES = 2;
struct EncvHalf {
  float xs[TQ_GROUP_TOK][ENCV_XS];     // the group's rows
  // unit vectors, [token][channel]: fp16 hi part, then lo part; once the rotation is done
  // the area holds the list, codes and products of the recomputation
  __half uh[2][TQ_GROUP_TOK][ENCV_UH];
  uint32_t img[256];
  float norm[TQ_GROUP_TOK];
  int wl_n;
  int pad_[3];
};
constexpr int ENCV_PI_BYTES = TQ_D * TQ_D * 2 * 2;  // fp16 hi and lo fragments of Pi
constexpr int ENCV_SMEM = ENCV_PI_BYTES + ENCV_HALVES * (int)sizeof(EncvHalf) + 128;
static_assert(TQ_D * TQ_GROUP_TOK * 3 + TQ_D * 4 * (TQ_D / 32) <= (int)sizeof(EncvHalf::uh),
              "the recomputation's list, codes and products fit in the unit-vector area");

template <int DT>
__global__ void __launch_bounds__(ENCV_HALVES* TQ_D, 2) encode_values_kernel(EncodeArgs a) {
  const tq_geom& g = a.g;
  const int e = threadIdx.x & (TQ_D - 1), half = threadIdx.x >> 7;
  const int wq = e >> 5, lane = e & 31, r = lane >> 2, c = lane & 3;
  const int groups = g.block_tokens_pad / TQ_GROUP_TOK;
  const int total = a.seq_count * g.n_kv_heads * a.max_new_blocks * groups;
  const int vb = g.value_bits;
  const int n_bnd = (1 << vb) - 1;

  extern __shared__ __align__(16) uint8_t encv_smem[];
  // Pi as A fragments: [16-channel tile][16-input-channel step][hi | lo][lane] x 16 bytes
  uint4* pif = (uint4*)encv_smem;
  EncvHalf* hs = (EncvHalf*)(encv_smem + ENCV_PI_BYTES) + half;
  // s_bnd[0] = -inf, s_bnd[1 + j] = boundary j, +inf beyond the last one: a coordinate with
  // code c lies in (s_bnd[c], s_bnd[c + 1]]
  float* s_bnd = (float*)(encv_smem + ENCV_PI_BYTES + ENCV_HALVES * sizeof(EncvHalf));
  auto half_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "n"(TQ_D) : "memory"); };
  const float* pi_rows = a.tables->pi;  // pi[ch][d]
  // whether every row of the caller's tensor starts on a 16-byte boundary (the ring's do)
  const bool keys = a.polar_keys_pass != 0;  // this launch encodes the keys (PolarQuant keys)
  const void* in_base = keys ? a.k : a.v;
  const void* ring_base = keys ? a.hot_k : a.hot_v;
  const int out_off = keys ? 0 : g.v_off, nrm_off = keys ? g.scale_off : g.norm_off;
  const bool rows_aligned = [&]() {
    const int64_t epc = 16 / (int64_t)sizeof(typename Elem<DT>::type);
    return ((uintptr_t)in_base & 15) == 0 && a.seq_stride % epc == 0 && a.tok_stride % epc == 0 &&
           a.head_stride % epc == 0;
  }();

  for (int idx = threadIdx.x; idx < 8 * 8 * 32; idx += ENCV_HALVES * TQ_D) {
    const int L = idx & 31, ks = (idx >> 5) & 7, MT = idx >> 8;
    const int ch0 = 16 * MT + (L >> 2), d0 = 16 * ks + 2 * (L & 3);
    // a0: (row r, k 2c..), a1: (row r+8, k 2c..), a2: (row r, k 2c+8..), a3: (row r+8, k 2c+8..)
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 p = *(const float2*)&pi_rows[(ch0 + 8 * (q & 1)) * TQ_D + d0 + 8 * (q >> 1)];
      __half h0, l0, h1, l1;
      split_h(p.x, h0, l0);
      split_h(p.y, h1, l1);
      hi[q] = h2_bits(h0, h1);
      lo[q] = h2_bits(l0, l1);
    }
    pif[((MT * 8 + ks) * 2 + 0) * 32 + L] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    pif[((MT * 8 + ks) * 2 + 1) * 32 + L] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
  if (threadIdx.x < 16) s_bnd[1 + threadIdx.x] = a.tables->boundaries[threadIdx.x];
  if (threadIdx.x == 16) s_bnd[0] = -INFINITY;
  if (threadIdx.x == 17) s_bnd[17] = INFINITY;
  __syncthreads();

  for (int w = blockIdx.x * ENCV_HALVES + half; w < total; w += gridDim.x * ENCV_HALVES) {
    int gq = w % groups;
    int rr = w / groups;
    int jb = rr % a.max_new_blocks;
    rr /= a.max_new_blocks;
    int head = rr % g.n_kv_heads;
    int seq = a.seq_begin + rr / g.n_kv_heads;
    const int n0 = a.seq_len[a.layer * g.n_seqs + seq];
    const int nb0 = n_cold_blocks(n0, g.hot_window, g.block_tokens);
    const int nb1 = n_cold_blocks(n0 + a.n_tokens, g.hot_window, g.block_tokens);
    const int blk = nb0 + jb;
    if (blk >= nb1) continue;  // uniform over the half
    const int S = g.block_tokens;
    const TokenSource<DT> src = make_source<DT>(a, ring_base, in_base, seq, head, n0);
    uint8_t* page = a.pages + page_offset(g, a.layer, seq, head, blk);

    // (No barrier here: the last reads of the previous item's rows, unit vectors and lists lie
    // before its last two barriers, and its image is overwritten only after three more.)
    if (e == 0) hs->wl_n = 0;
    {
      // The group's 16 rows are consecutive positions: the ring slot of the first one is worked
      // out once (one division), the others follow by increments.  Rows past the end of the
      // block (a block length that is no multiple of 16) read the block's last row and count
      // as zero.
      using T = typename Elem<DT>::type;
      const int tok0 = gq * TQ_GROUP_TOK, pos0 = blk * S + tok0;
      const int ring0 = pos0 % src.cap;
      auto row_of = [&](int t) -> const T* {  // token t of the group (clamped)
        const int te = min(t, S - 1 - tok0);
        const int pos = pos0 + te;
        int ri = ring0 + te;
        ri -= ri >= src.cap ? src.cap : 0;
        return pos < n0 ? (const T*)src.ring + (size_t)ri * TQ_D
                        : (const T*)src.in + (size_t)(pos - n0) * src.tok_stride;
      };
      if (rows_aligned) {
        // 16-byte pieces, all requested before the first is used
        constexpr int EPC = 16 / (int)sizeof(T), CH = TQ_D / EPC, NCH = TQ_GROUP_TOK * CH / TQ_D;
        uint4 raw[NCH];
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int id = e + TQ_D * i;
          raw[i] = *(const uint4*)(row_of(id / CH) + (id % CH) * EPC);
        }
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int id = e + TQ_D * i, t = id / CH, c0 = (id % CH) * EPC;
          const bool live = tok0 + t < S;
          const T* pv = (const T*)&raw[i];
          float f[EPC];
#pragma unroll
          for (int k = 0; k < EPC; ++k) f[k] = live ? Elem<DT>::ld(pv, k) : 0.0f;
#pragma unroll
          for (int k = 0; k < EPC; k += 4)
            *(float4*)&hs->xs[t][c0 + k] = make_float4(f[k], f[k + 1], f[k + 2], f[k + 3]);
        }
      } else {
        float xv[TQ_GROUP_TOK];
#pragma unroll
        for (int t = 0; t < TQ_GROUP_TOK; ++t) xv[t] = Elem<DT>::ld(row_of(t), e);
#pragma unroll
        for (int t = 0; t < TQ_GROUP_TOK; ++t) hs->xs[t][e] = tok0 + t < S ? xv[t] : 0.0f;
      }
    }
    half_sync();
    {  // norms: 8 threads per token, accumulator j sums elements j, j+8, j+16, ...
      const int t = e >> 3, j = e & 7;
      float xr[TQ_D / 8];
#pragma unroll
      for (int i = 0; i < TQ_D / 8; ++i) xr[i] = hs->xs[t][8 * i + j];
      float sq = __fmul_rn(xr[0], xr[0]);
#pragma unroll
      for (int i = 1; i < TQ_D / 8; ++i) sq = __fadd_rn(sq, __fmul_rn(xr[i], xr[i]));
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 1));  // (r0+r1), (r2+r3), ...
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 2));  // (r0+r1)+(r2+r3), ...
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 4));
      const float nrm = __fsqrt_rn(sq);  // (the same bits in all eight threads of the token)
      if (j == 0) {
        hs->norm[t] = nrm;
        ((float*)(page + nrm_off))[gq * TQ_GROUP_TOK + t] = nrm;
      }
      // unit vectors as fp16 hi / lo parts, [token][channel].  The tensor-core rotation only
      // has to land within the slack, so it takes x * (1 / norm), one or two units in the
      // last place from the reference's x / norm; the recomputation divides.
      const float inv = 1.0f / fmaxf(nrm, 1e-30f);
#pragma unroll
      for (int i = 0; i < TQ_D / 8; ++i) {
        __half h, l;
        split_h(xr[i] * inv, h, l);
        hs->uh[0][t][8 * i + j] = h;
        hs->uh[1][t][8 * i + j] = l;
      }
    }
    half_sync();
    // Rotation.  y[mt][nt][i]: channel 32 wq + 16 mt + r + 8 (i >> 1), token 8 nt + 2c + (i & 1)
    float y[2][2][4];
    {
      float cx[2][2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) y[mt][nt][i] = cx[mt][nt][i] = 0.0f;
      // lanes 8m .. 8m+7 address the rows of matrix m: tokens 8 (m >> 1) + 0..7, input
      // channels 16 ks + 8 (m & 1) + 0..7; the four matrices are the B fragments {b0, b1} of
      // the two 8-token tiles
      const int m_tok = 8 * (lane >> 4) + (lane & 7), m_d = 8 * ((lane >> 3) & 1);
      const uint32_t ub_hi = (uint32_t)__cvta_generic_to_shared(&hs->uh[0][m_tok][m_d]);
      const uint32_t ub_lo = (uint32_t)__cvta_generic_to_shared(&hs->uh[1][m_tok][m_d]);
      const uint4* pa = pif + (size_t)(2 * wq) * 8 * 2 * 32 + lane;
#pragma unroll 2
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t bh[4], bl[4];
        enc_ldsm_x4(bh, ub_hi + ks * 32);
        enc_ldsm_x4(bl, ub_lo + ks * 32);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const uint4 ah = pa[((mt * 8 + ks) * 2 + 0) * 32], al = pa[((mt * 8 + ks) * 2 + 1) * 32];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            enc_mma16816(y[mt][nt], ah, bh[2 * nt], bh[2 * nt + 1]);
            enc_mma16816(cx[mt][nt], ah, bl[2 * nt], bl[2 * nt + 1]);
            enc_mma16816(cx[mt][nt], al, bh[2 * nt], bh[2 * nt + 1]);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i)
            y[mt][nt][i] = fmaf(cx[mt][nt][i], 1.0f / 2048.0f, y[mt][nt][i]);
    }
    // code = number of boundaries below the coordinate (one boundary load serves the lane's 16
    // coordinates); a coordinate with a boundary within the slack is done again.
    // Coordinate k = 8 mt + 4 nt + i of the lane.
    // (the boundaries ascend, so the count is found by bisection: value_bits comparisons)
    int code[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) code[k] = 0;
    for (int step = (n_bnd + 1) >> 1; step > 0; step >>= 1) {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        code[k] += (s_bnd[code[k] + step] < y[k >> 3][(k >> 2) & 1][k & 3]) ? step : 0;
    }
    unsigned redo = 0u;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float yy = y[k >> 3][(k >> 2) & 1][k & 3];
      const float below = s_bnd[code[k]], above = s_bnd[code[k] + 1];
      redo |= (yy - below < ROT_SLACK || above - yy < ROT_SLACK) ? (1u << k) : 0u;
    }
    // The coordinates to be done again (a handful per group) go on a list in the unit-vector
    // area, which is free by now; the half's four warps take them in turn.  A warp computes
    // the 128 products of one coordinate in parallel (four per lane, the unit vector formed
    // again from the row by the same division) and one lane adds them up in the reference's
    // order from shared memory.
    {
      unsigned short* wl = (unsigned short*)&hs->uh[0][0][0];             // (channel, token) items
      unsigned char* fixed = (unsigned char*)(wl + TQ_D * TQ_GROUP_TOK);   // [token][channel] codes
      float* prod = (float*)(fixed + TQ_D * TQ_GROUP_TOK) + wq * TQ_D;     // this warp's products
      half_sync();  // every warp is done with the unit vectors (the list's counter was zeroed
                    // at the top of the item, two barriers ago)
      unsigned todo = redo;
      while (todo) {
        const int k = __ffs((int)todo) - 1;
        todo &= todo - 1;
        const int ch = 32 * wq + 16 * (k >> 3) + r + 8 * ((k >> 1) & 1);
        const int t = 8 * ((k >> 2) & 1) + 2 * c + (k & 1);
        wl[atomicAdd(&hs->wl_n, 1)] = (unsigned short)(ch | (t << 8));
      }
      half_sync();
      const int n_items = hs->wl_n;
      for (int it = wq; it < n_items; it += TQ_D / 32) {
        const int item = wl[it], c2 = item & 255, t2 = item >> 8;
        const float safe = fmaxf(hs->norm[t2], 1e-30f);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int dd = 32 * k + lane;
          prod[dd] = __fmul_rn(__fdiv_rn(hs->xs[t2][dd], safe), __ldg(&pi_rows[c2 * TQ_D + dd]));
        }
        __syncwarp();
        if (lane == 0) {
          float4 p4 = *(const float4*)&prod[0];
          float yy = __fadd_rn(__fadd_rn(__fadd_rn(p4.x, p4.y), p4.z), p4.w);
#pragma unroll 8
          for (int q = 1; q < TQ_D / 4; ++q) {
            p4 = *(const float4*)&prod[4 * q];
            yy = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(yy, p4.x), p4.y), p4.z), p4.w);
          }
          int cd = 0;
          for (int j = 0; j < n_bnd; ++j) cd += (s_bnd[1 + j] < yy) ? 1 : 0;
          fixed[t2 * TQ_D + c2] = (unsigned char)cd;
        }
        __syncwarp();
      }
      half_sync();
      while (redo) {
        const int k = __ffs((int)redo) - 1;
        redo &= redo - 1;
        const int ch = 32 * wq + 16 * (k >> 3) + r + 8 * ((k >> 1) & 1);
        const int t = 8 * ((k >> 2) & 1) + 2 * c + (k & 1);
        const int cd = fixed[t * TQ_D + ch];
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) code[kk] = kk == k ? cd : code[kk];
      }
    }
    // The lane's codes are pairs 4 MT .. 4 MT + 3 of its own lane record (MT = 2 wq + mt):
    // (channel r, tokens 2c, 2c+1), (r, 2c+8, 2c+9), (r + 8, 2c, 2c+1), (r + 8, 2c+8, 2c+9);
    // every byte of the group image is written by exactly one lane.
    uint8_t* img = (uint8_t*)hs->img;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const int MT = 2 * wq + mt;
      // pair q = 2 h + nt holds coordinates k = 8 mt + 4 nt + 2 h, + 1
      if (vb == 4) {
        uint32_t wv = 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int k = 8 * mt + 4 * (q & 1) + 2 * (q >> 1);
          wv |= (uint32_t)(code[k] | (code[k + 1] << 4)) << (8 * q);
        }
        *(uint32_t*)(img + v_record_byte_off(4, lane, 4 * MT)) = wv;
      } else {
        uint32_t wv = 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int k = 8 * mt + 4 * (q & 1) + 2 * (q >> 1);
          wv |= (uint32_t)(code[k] | (code[k + 1] << 3)) << (6 * q);
        }
#pragma unroll
        for (int bq = 0; bq < 3; ++bq)
          img[v_record_byte_off(3, lane, 3 * MT + bq)] = (uint8_t)(wv >> (8 * bq));
      }
    }
    half_sync();
    uint32_t* dst = (uint32_t*)(page + out_off + (size_t)gq * v_group_bytes(vb));
    const int words = v_group_bytes(vb) / 4;
    for (int i = e; i < words; i += TQ_D) dst[i] = hs->img[i];
  }
}

// ---------------------------------------------------------------------------------------
// The same value encoder with the rotation on the fifth-generation tensor cores: both operands
// of Y^T = Pi . U^T live in shared memory, so the products are issued by one thread as
// tcgen05.mma instructions (M = 128 channels, N = 16 tokens, K = 16 per instruction) with the
// accumulators in tensor memory, and every thread reads back the 16 tokens of its own channel
// with tcgen05.ld.  Operand split and slack are those of the kernel above.
//
// Shared-memory operands are K-major without swizzling: 8 x 8 core matrices of 16-bit values
// (8 rows of 16 bytes, 128 bytes each), "stride" 128 bytes to the next eight rows and
// "leading" offset to the core matrix of the next eight input channels.  Pi (hi and lo parts)
// is laid out once per CTA, the unit vectors per group.
//
// One CTA per SM: ENC5_PARTS independent parts of 128 threads share the copy of Pi.  A part
// has three groups in flight: while the tensor cores rotate group i + 1 (into the other half
// of the part's 64 columns of tensor memory) and the rows of group i + 2 are on their way
// from global memory, its threads turn the products of group i into codes.
//
// A product that lies within the slack of a boundary is not recomputed on the spot: the part
// puts (row, destination, norm, channel, token, code) on a list, and the list is worked off
// when the part has run out of groups (or the list is full): a thread per entry computes the
// exact sum in the reference's order and, where the code differs, flips the bits of the code in
// the page.  The main loop then has three barriers per group and no serial tail.  All waits
// are bounded.
// ---------------------------------------------------------------------------------------
TQ_DEV uint32_t enc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
TQ_DEV uint64_t umma_desc_k_major(uint32_t saddr, uint32_t leading_bytes, uint32_t stride_bytes) {
  // start address, leading and stride byte offsets in 16-byte units; descriptor version 1;
  // base offset 0, no swizzle
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((stride_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128, N = 16
constexpr uint32_t UMMA_IDESC_M128_N16 = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
TQ_DEV void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(UMMA_IDESC_M128_N16), "r"(accumulate)
      : "memory");
}
TQ_DEV void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
TQ_DEV void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

#ifndef TQ_ENC5_PARTS
#define TQ_ENC5_PARTS 6
#endif
constexpr int ENC5_PARTS = TQ_ENC5_PARTS;
constexpr int ENC5_LIST = 160;  // entries of a part's list
struct Enc5Info {                 // what the later phases need to know about a group
  const void* rowp[TQ_GROUP_TOK];  // where each token's row comes from (null: padding)
  uint32_t* dst;                   // the group's codes in the page
  float* nrm_dst;                  // the group's norms in the page
  float norm[TQ_GROUP_TOK];
};
struct Enc5Part {
  float xs[TQ_GROUP_TOK][ENCV_XS];  // the rows of the group being staged
  // its unit vectors as tensor-core operands, hi then lo part: [K / 8][2 token groups][8][8]
  __align__(16) __half ub[2][TQ_GROUP_TOK * TQ_D];
  uint32_t img[256];              // the codes of the group being packed
  Enc5Info info[3];               // group m uses info[m % 3]
  unsigned long long bar[2];      // "the products of group m are done": bar[m & 1]
  const void* l_row[ENC5_LIST];   // the list
  uint32_t* l_dst[ENC5_LIST];
  float l_norm[ENC5_LIST];
  uint32_t l_meta[ENC5_LIST];     // channel | token << 8 | code << 12
  int l_cnt;                      // appends tried (may exceed the capacity)
  int pad_[3];
};
static_assert(sizeof(Enc5Part) % 16 == 0, "16-byte operands");
constexpr int ENC5_SMEM = ENCV_PI_BYTES + ENC5_PARTS * (int)sizeof(Enc5Part) + 320;
static_assert(ENC5_SMEM <= 227 * 1024, "shared memory of one CTA");
constexpr int ENC5_TMEM_COLS = ENC5_PARTS * 64 <= 256 ? 256 : 512;  // (a power of two)
static_assert(ENC5_PARTS * 64 <= ENC5_TMEM_COLS, "tensor memory of one SM");
constexpr int ENC5_WAIT = 1 << 16;  // probes of a product barrier before a wait gives up

template <int DT, int VB>
__global__ void __launch_bounds__(ENC5_PARTS* TQ_D, 1) encode_values_tc5_kernel(EncodeArgs a) {
  using T = typename Elem<DT>::type;
  constexpr int EPC = 16 / (int)sizeof(T), CH = TQ_D / EPC, NCH = TQ_GROUP_TOK * CH / TQ_D;
  const tq_geom& g = a.g;
  const int e = threadIdx.x & (TQ_D - 1), part = threadIdx.x >> 7;
  const int wq = e >> 5, lane = e & 31;
  const int groups = g.block_tokens_pad / TQ_GROUP_TOK;
  const int total = a.seq_count * g.n_kv_heads * a.max_new_blocks * groups;
  constexpr int vb = VB;  // bits of a code (the launcher picks the instance)
  constexpr int n_bnd = (1 << vb) - 1;
  const int S = g.block_tokens;

  extern __shared__ __align__(128) uint8_t enc5_smem[];
  __half* pa = (__half*)enc5_smem;  // Pi: [hi | lo][K / 8][M / 8][8][8] fp16
  Enc5Part* ps = (Enc5Part*)(enc5_smem + ENCV_PI_BYTES) + part;
  float* s_bnd = (float*)(enc5_smem + ENCV_PI_BYTES + ENC5_PARTS * sizeof(Enc5Part));
  float2* s_bp = (float2*)(s_bnd + 32);  // (boundary below, boundary above) of each code
  uint32_t* s_tmem = (uint32_t*)(s_bp + 18);
  auto part_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + part), "n"(TQ_D) : "memory"); };
  const float* pi_rows = a.tables->pi;  // pi[ch][d]
  const bool keys = a.polar_keys_pass != 0;
  const void* in_base = keys ? a.k : a.v;
  const void* ring_base = keys ? a.hot_k : a.hot_v;
  const int out_off = keys ? 0 : g.v_off, nrm_off = keys ? g.scale_off : g.norm_off;
  const bool rows_aligned = [&]() {
    const int64_t epc = EPC;
    return ((uintptr_t)in_base & 15) == 0 && a.seq_stride % epc == 0 && a.tok_stride % epc == 0 &&
           a.head_stride % epc == 0;
  }();

  // Pi as the A operand: element (ch, d) of part p at
  // p * 32 KB + ((d / 8) * 16 + ch / 8) * 128 + (ch % 8) * 16 + (d % 8) * 2 bytes
  for (int idx = threadIdx.x; idx < TQ_D * TQ_D / 2; idx += ENC5_PARTS * TQ_D) {
    const int ch = idx >> 6, d = (idx & 63) * 2;
    const float2 p = *(const float2*)&pi_rows[ch * TQ_D + d];
    __half h0, l0, h1, l1;
    split_h(p.x, h0, l0);
    split_h(p.y, h1, l1);
    const int off = ((d >> 3) * 16 + (ch >> 3)) * 64 + (ch & 7) * 8 + (d & 7);  // in halves
    *(uint32_t*)&pa[off] = h2_bits(h0, h1);
    *(uint32_t*)&pa[TQ_D * TQ_D + off] = h2_bits(l0, l1);
  }
  if (threadIdx.x < 16) s_bnd[1 + threadIdx.x] = a.tables->boundaries[threadIdx.x];
  if (threadIdx.x == 16) s_bnd[0] = -INFINITY;
  if (threadIdx.x == 17) s_bnd[17] = INFINITY;
  if (threadIdx.x >= 32 && threadIdx.x < 32 + 17) {
    const int c = threadIdx.x - 32;  // code c lies between boundaries c - 1 and c
    s_bp[c] = make_float2(c == 0 ? -INFINITY : a.tables->boundaries[c - 1],
                          c == 16 ? INFINITY : a.tables->boundaries[c]);
  }
  int* s_step = (int*)(s_tmem + 1);  // the distance between a part's groups, as four indices
  if (threadIdx.x == 18) {
    int w = gridDim.x * ENC5_PARTS;
    s_step[0] = w % groups, w /= groups;
    s_step[1] = w % a.max_new_blocks, w /= a.max_new_blocks;
    s_step[2] = w % g.n_kv_heads, s_step[3] = w / g.n_kv_heads;
  }
  if (e == 2) ps->l_cnt = 0;
  if (e < 2) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(enc_smem(&ps->bar[e])), "r"(1)
                 : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {  // one warp allocates the CTA's tensor memory ...
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(enc_smem(s_tmem)),
                 "r"(ENC5_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // Pi is read by the tensor cores
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *(volatile uint32_t*)s_tmem + (uint32_t)(part * 64);  // this part's columns
  const uint32_t pa_addr = enc_smem(pa);
  const uint32_t ub_addr = enc_smem(&ps->ub[0][0]);

  bool gave_up = false;
  // bounded wait for the products of group m
  auto wait_products = [&](int m) {
    if (gave_up) return;
    const uint32_t bar = enc_smem(&ps->bar[m & 1]);
    const unsigned parity = (unsigned)((m >> 1) & 1);
    int n = 0;
    unsigned done = 0;
    while (!done) {
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}\n"
          : "=r"(done)
          : "r"(bar), "r"(parity)
          : "memory");
      if (!done && ++n >= ENC5_WAIT) {
        atomicOr(a.status, TQ_STATUS_WAIT_TIMEOUT);
        gave_up = true;  // (no later wait of this thread probes again)
        break;
      }
    }
  };

  // the groups of this part, in order: group number w = ((seq * heads + head) * blocks + jb) *
  // groups + gq, w = first, first + step, ...; the four indices are kept and stepped with
  // carries (no division per group); a group whose block this call does not flush is skipped
  int gq_n, jb_n, head_n, seq_n;       // the next candidate (seq_n counts from seq_begin)
  // (the step, in the same mixed radix, is s_step)
  {
    int w = blockIdx.x * ENC5_PARTS + part;
    gq_n = w % groups, w /= groups;
    jb_n = w % a.max_new_blocks, w /= a.max_new_blocks;
    head_n = w % g.n_kv_heads, seq_n = w / g.n_kv_heads;
  }
  int seq_known = -1, n0_known = 0, nb0_known = 0, nb1_known = 0, r0_known = 0;  // per sequence
  uint4 raw[NCH];                    // this thread's 16-byte pieces of the next group's rows
  int lim_raw = 0;                   // ... and how many of its tokens lie inside the block
  // finds group m, notes what the later phases need in info[m % 3] and starts the loads of its
  // rows; false when the part has run out of groups
  auto advance = [&](int m) -> bool {
    while (seq_n < a.seq_count) {
      const int gq = gq_n, jb = jb_n, head = head_n, seq = a.seq_begin + seq_n;
      {  // step to the next candidate
        gq_n += s_step[0];
        int c = gq_n >= groups ? 1 : 0;
        gq_n -= c ? groups : 0;
        jb_n += s_step[1] + c;
        c = jb_n >= a.max_new_blocks ? 1 : 0;
        jb_n -= c ? a.max_new_blocks : 0;
        head_n += s_step[2] + c;
        c = head_n >= g.n_kv_heads ? 1 : 0;
        head_n -= c ? g.n_kv_heads : 0;
        seq_n += s_step[3] + c;
      }
      if (seq != seq_known) {
        n0_known = a.seq_len[a.layer * g.n_seqs + seq];
        nb0_known = n_cold_blocks(n0_known, g.hot_window, g.block_tokens);
        nb1_known = n_cold_blocks(n0_known + a.n_tokens, g.hot_window, g.block_tokens);
        r0_known = n0_known % g.hot_cap;
        seq_known = seq;
      }
      const int n0 = n0_known;
      const int blk = nb0_known + jb;
      if (blk >= nb1_known) continue;
      const TokenSource<DT> src = make_source<DT>(a, ring_base, in_base, seq, head, n0);
      const int lim = S - gq * TQ_GROUP_TOK;  // tokens of the group inside the block
      lim_raw = lim;
      const int pos0 = blk * S + gq * TQ_GROUP_TOK;
      // ring slot of position pos0 (used for positions below n0, which lie less than the
      // ring's capacity below it)
      int ring0 = r0_known + (pos0 - n0);
      ring0 += ring0 < 0 ? src.cap : 0;
      if (ring0 < 0 || ring0 >= src.cap) ring0 = pos0 % src.cap;
      auto row_of = [&](int t) -> const T* {  // token t of the group (clamped)
        const int te = min(t, lim - 1);
        const int pos = pos0 + te;
        int ri = ring0 + te;
        ri -= ri >= src.cap ? src.cap : 0;
        return pos < n0 ? (const T*)src.ring + (size_t)ri * TQ_D
                        : (const T*)src.in + (size_t)(pos - n0) * src.tok_stride;
      };
      if (rows_aligned) {
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int id = e + TQ_D * i;
          raw[i] = *(const uint4*)(row_of(id / CH) + (id % CH) * EPC);
        }
      }
      Enc5Info* nf = &ps->info[m % 3];
      uint8_t* page = a.pages + page_offset(g, a.layer, seq, head, blk);
      if (e < TQ_GROUP_TOK) nf->rowp[e] = e < lim ? (const void*)row_of(e) : nullptr;
      if (e == 64) {
        nf->dst = (uint32_t*)(page + out_off + (size_t)gq * v_group_bytes(vb));
        nf->nrm_dst = (float*)(page + nrm_off) + gq * TQ_GROUP_TOK;
      }
      return true;
    }
    return false;
  };

  // group m (rows in `raw` if the rows are aligned): rows, norms, unit vectors, and the
  // products started
  auto stage_in = [&](int m) {
    Enc5Info* nf = &ps->info[m % 3];
    if (rows_aligned) {
#pragma unroll
      for (int i = 0; i < NCH; ++i) {
        const int id = e + TQ_D * i, t = id / CH, c0 = (id % CH) * EPC;
        const T* pv = (const T*)&raw[i];
        float f[EPC];
#pragma unroll
        for (int k = 0; k < EPC; ++k) f[k] = Elem<DT>::ld(pv, k);
        if (t >= lim_raw) {  // padding (only in a block's last group)
#pragma unroll
          for (int k = 0; k < EPC; ++k) f[k] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < EPC; k += 4)
          *(float4*)&ps->xs[t][c0 + k] = make_float4(f[k], f[k + 1], f[k + 2], f[k + 3]);
      }
    } else {
      part_sync();  // (the row pointers were written by other threads)
      float xv[TQ_GROUP_TOK];
#pragma unroll
      for (int t = 0; t < TQ_GROUP_TOK; ++t) {
        const T* row = (const T*)nf->rowp[t];
        xv[t] = row != nullptr ? Elem<DT>::ld(row, e) : 0.0f;
      }
#pragma unroll
      for (int t = 0; t < TQ_GROUP_TOK; ++t) ps->xs[t][e] = xv[t];
    }
    part_sync();
    ps->img[e] = 0u;
    ps->img[e + 128] = 0u;
    const int t = e >> 3, j = e & 7;
    float xr[TQ_D / 8];
    float inv;
    {  // norms (numpy's 8-accumulator order)
#pragma unroll
      for (int i = 0; i < TQ_D / 8; ++i) xr[i] = ps->xs[t][8 * i + j];
      float sq = __fmul_rn(xr[0], xr[0]);
#pragma unroll
      for (int i = 1; i < TQ_D / 8; ++i) sq = __fadd_rn(sq, __fmul_rn(xr[i], xr[i]));
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 1));
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 2));
      sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, 4));
      const float nrm = __fsqrt_rn(sq);
      if (j == 0) {
        nf->norm[t] = nrm;
        nf->nrm_dst[t] = nrm;
      }
      inv = 1.0f / fmaxf(nrm, 1e-30f);
    }
    // the operand area is read by the products of group m - 1 until they are done
    if (m > 0) wait_products(m - 1);
    // the unit vectors as the B operand: element (token t, channel d) of part p at
    // p * 4 KB + ((d / 8) * 2 + t / 8) * 128 + (t % 8) * 16 + (d % 8) * 2 bytes
#pragma unroll
    for (int i = 0; i < TQ_D / 8; ++i) {
      __half h, l;
      split_h(xr[i] * inv, h, l);
      const int off = (i * 2 + (t >> 3)) * 64 + (t & 7) * 8 + j;  // in halves
      ps->ub[0][off] = h;
      ps->ub[1][off] = l;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // ... read by the tensor cores
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    part_sync();
    if (e == 32) {  // (a thread of the second warp: the first one notes the rows of the next group)
      // hi*hi into columns 0-15, hi*lo + lo*hi into columns 16-31; eight K steps each
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_main = tmem + (uint32_t)((m & 1) * 32);
      // the descriptors of K step kb are those of step 0 with the start address (in 16-byte
      // units, the low 14 bits; shared memory ends below 2^18) moved on by 4 KB (Pi) or 512
      // bytes (unit vectors)
      const uint64_t a_hi0 = umma_desc_k_major(pa_addr, 2048, 128);
      const uint64_t a_lo0 = umma_desc_k_major(pa_addr + TQ_D * TQ_D * 2, 2048, 128);
      const uint64_t b_hi0 = umma_desc_k_major(ub_addr, 256, 128);
      const uint64_t b_lo0 = umma_desc_k_major(ub_addr + TQ_GROUP_TOK * TQ_D * 2, 256, 128);
#pragma unroll
      for (int kb = 0; kb < 8; ++kb) {
        const uint64_t a_hi = a_hi0 + (uint64_t)(kb * (4096 >> 4));
        const uint64_t a_lo = a_lo0 + (uint64_t)(kb * (4096 >> 4));
        const uint64_t b_hi = b_hi0 + (uint64_t)(kb * (512 >> 4));
        const uint64_t b_lo = b_lo0 + (uint64_t)(kb * (512 >> 4));
        umma_f16_ss(d_main, a_hi, b_hi, kb > 0);
        umma_f16_ss(d_main + 16, a_hi, b_lo, kb > 0);
        umma_f16_ss(d_main + 16, a_lo, b_hi, 1u);
      }
      umma_commit(enc_smem(&ps->bar[m & 1]));
    }
  };

  // tokens `bits` (of tokens t0 .. t0 + 7) of channel `ch` of a group go on the list; returns
  // the ones that did not fit
  auto list_add = [&](const Enc5Info* nf, unsigned bits, uint32_t packed, int t0, int ch) {
    unsigned left = 0u;
    while (bits) {
      const int t = __ffs((int)bits) - 1;
      bits &= bits - 1;
      const void* row = nf->rowp[t0 + t];
      if (row == nullptr) continue;  // padding: all zeros, the products are exact
      const int i = atomicAdd(&ps->l_cnt, 1);
      if (i < ENC5_LIST) {
        ps->l_row[i] = row;
        ps->l_dst[i] = nf->dst;
        ps->l_norm[i] = nf->norm[t0 + t];
        ps->l_meta[i] =
            (uint32_t)ch | ((uint32_t)(t0 + t) << 8) | (((packed >> (4 * t)) & 15u) << 12);
      } else {
        left |= 1u << t;
      }
    }
    return left;
  };
  // the first n entries of the list, one per thread: exact sum in the reference's order (the
  // quotients and products rounded one by one, added up in sequence), the code it gives, and
  // the difference to the stored code flipped in the page.  Ends with the list empty; every
  // thread of the part calls it.
  auto list_flush = [&](int n) {
    for (int i = e; i < n; i += TQ_D) {
      const T* row = (const T*)ps->l_row[i];
      const uint32_t meta = ps->l_meta[i];
      const int c2 = (int)(meta & 255u), t2 = (int)((meta >> 8) & 15u);
      const float safe = fmaxf(ps->l_norm[i], 1e-30f);
      const float* pr = pi_rows + c2 * TQ_D;
      float yy = 0.0f;
#pragma unroll 2
      for (int d0 = 0; d0 < TQ_D; d0 += 8) {
        float x[8];
        if (rows_aligned) {
          uint4 rw[8 / EPC];
#pragma unroll
          for (int k = 0; k < 8 / EPC; ++k) rw[k] = *(const uint4*)(row + d0 + k * EPC);
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] = Elem<DT>::ld((const T*)rw, k);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] = Elem<DT>::ld(row, d0 + k);
        }
        const float4 pa4 = __ldg((const float4*)(pr + d0)), pb4 = __ldg((const float4*)(pr + d0 + 4));
        const float pv[8] = {pa4.x, pa4.y, pa4.z, pa4.w, pb4.x, pb4.y, pb4.z, pb4.w};
        float pd[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) pd[k] = __fmul_rn(__fdiv_rn(x[k], safe), pv[k]);
        // ((p0 + p1) + p2) + ... : the first product starts the sum
        yy = d0 == 0 ? pd[0] : __fadd_rn(yy, pd[0]);
#pragma unroll
        for (int k = 1; k < 8; ++k) yy = __fadd_rn(yy, pd[k]);
      }
      int cd = 0;
      for (int j = 0; j < n_bnd; ++j) cd += (s_bnd[1 + j] < yy) ? 1 : 0;
      const uint32_t delta = (uint32_t)cd ^ (meta >> 12);
      if (delta) {
        const int l = v_lane(t2, c2), bit = 2 * vb * v_pair(t2, c2) + vb * (t2 & 1);
        const uint32_t v = delta << (bit & 7);
        uint32_t* d32 = ps->l_dst[i];
        const int off0 = v_record_byte_off(vb, l, bit >> 3);
        if (v & 255u) atomicXor(&d32[off0 >> 2], (v & 255u) << ((off0 & 3) * 8));
        if (v >> 8) {
          const int off1 = v_record_byte_off(vb, l, (bit >> 3) + 1);
          atomicXor(&d32[off1 >> 2], (v >> 8) << ((off1 & 3) * 8));
        }
      }
    }
    part_sync();
    if (e == 0) ps->l_cnt = 0;
    part_sync();
  };

  // group m: products -> codes -> the page
  auto stage_out = [&](int m) {
    const Enc5Info* nf = &ps->info[m % 3];
    wait_products(m);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // thread e owns channel e: codes of its 16 tokens, eight at a time, by bisection; a token
    // whose product lies within the slack of a boundary goes on the list
    const int ch = 32 * wq + lane;
    const int dq = ch & 7, i16 = ch >> 3;  // record lane group and slot of this thread's channel
    uint32_t* img = ps->img;
    unsigned redo[2];
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float y[8];
      {
        float cx[8];
        const uint32_t taddr =
            tmem + (uint32_t)((m & 1) * 32 + 8 * h) + ((uint32_t)(32 * wq) << 16);
        tmem_ld8(taddr, y);
        tmem_ld8(taddr + 16, cx);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 8; ++t) y[t] = fmaf(cx[t], 1.0f / 2048.0f, y[t]);
      }
      int code[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) code[t] = 0;
      for (int step = (n_bnd + 1) >> 1; step > 0; step >>= 1) {
#pragma unroll
        for (int t = 0; t < 8; ++t) code[t] += (s_bnd[code[t] + step] < y[t]) ? step : 0;
      }
      unsigned rd = 0u;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float2 ba = s_bp[code[t]];
        rd |= (y[t] - ba.x < ROT_SLACK || ba.y - y[t] < ROT_SLACK) ? (1u << t) : 0u;
      }
      uint32_t pk = 0u;  // the codes as computed, a nibble each: for the list and the 4-bit image
      if (vb == 4 || rd) {
#pragma unroll
        for (int t = 0; t < 8; ++t) pk |= (uint32_t)code[t] << (4 * t);
      }
      packed[h] = pk;
      redo[h] = rd ? list_add(nf, rd, pk, 8 * h, ch) : 0u;
      // this channel's 4 token pairs into the group image
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int l = dq * 4 + c, p = 2 * i16 + h;
        if (vb == 4) {
          ((uint8_t*)img)[v_record_byte_off(4, l, p)] = (uint8_t)((pk >> (8 * c)) & 255u);
        } else {
          const uint32_t f = (uint32_t)(code[2 * c] | (code[2 * c + 1] << 3));
          const int bit = 6 * p, wd = bit >> 5, sh = bit & 31;
          atomicOr(&img[((wd >> 1) * 256 + l * 8 + (wd & 1) * 4) >> 2], f << sh);
          if (sh > 26)
            atomicOr(&img[((((wd + 1) >> 1)) * 256 + l * 8 + ((wd + 1) & 1) * 4) >> 2],
                     f >> (32 - sh));
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    part_sync();
    uint32_t* dst = nf->dst;
    const int words = v_group_bytes(vb) / 4;
    for (int i = e; i < words; i += TQ_D) dst[i] = img[i];
    // (the image is zeroed again after the first barrier of the next group's staging)
    int tried = ps->l_cnt;  // the same for every thread: nobody appends before the next group
    while (tried > ENC5_LIST) {  // some entries did not fit: work the list off and try again
      part_sync();               // (the group's codes are in the page)
      list_flush(ENC5_LIST);
#pragma unroll
      for (int h = 0; h < 2; ++h)
        if (redo[h]) redo[h] = list_add(nf, redo[h], packed[h], 8 * h, ch);
      part_sync();
      tried = ps->l_cnt;
    }
  };

  int m = 0;  // groups staged so far
  bool more = advance(0);
  while (more) {
    stage_in(m);
    more = advance(m + 1);
    if (m > 0) stage_out(m - 1);
    ++m;
  }
  if (m > 0) {
    if (m > 1) {  // (the image still holds the codes of group m - 2)
      part_sync();
      ps->img[e] = 0u;
      ps->img[e + 128] = 0u;
      part_sync();
    }
    stage_out(m - 1);
  }
  part_sync();  // the last group's codes are in the page
  list_flush(min(ps->l_cnt, ENC5_LIST));

  // ... and the same warp gives the tensor memory back
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*(volatile uint32_t*)s_tmem),
                 "r"(ENC5_TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// Hot-ring writer: the new tokens that stay uncompressed go to slot (position % hot_cap).
// grid = (tokens, heads, seqs); token index counts back from the newest.  The CTA that
// finishes last then adds the new tokens to the sequence lengths: every kernel of the append
// (the encoders before this one in the stream, and every CTA of this one) has read the old
// lengths by then.  The kernel may be launched with programmatic stream serialization: it
// waits for the kernel before it in the stream before it reads or writes anything.
// ---------------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(TQ_D) ring_write_kernel(EncodeArgs a) {
  using T = typename Elem<DT>::type;
  const tq_geom& g = a.g;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int seq = a.seq_begin + blockIdx.z;
  const int head = blockIdx.y;
  const int n0 = a.seq_len[a.layer * g.n_seqs + seq];
  const int n1 = n0 + a.n_tokens;
  const int pos = n1 - 1 - (int)blockIdx.x;
  const int hot_start = n_cold_blocks(n1, g.hot_window, g.block_tokens) * g.block_tokens;
  if (pos >= n0 && pos >= hot_start) {
    const size_t in = (size_t)(seq - a.seq_begin) * a.seq_stride +
                      (size_t)(pos - n0) * a.tok_stride + (size_t)head * a.head_stride + threadIdx.x;
    const size_t out =
        hot_offset_elems(g, a.layer, seq, head) + (size_t)(pos % g.hot_cap) * TQ_D + threadIdx.x;
    ((T*)a.hot_k)[out] = ((const T*)a.k)[in];
    ((T*)a.hot_v)[out] = ((const T*)a.v)[in];
  }
  // last CTA out: the counter sits in the status word's 256-byte block and returns to zero
  __shared__ int s_last;
  __syncthreads();  // every thread of the CTA has read its length
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd((unsigned*)a.status + 16, 1u);
    s_last = prev == total - 1;
    if (s_last) {
      ((unsigned*)a.status)[16] = 0u;
      __threadfence();
    }
  }
  __syncthreads();
  if (s_last) {
    for (int i = threadIdx.x; i < a.seq_count; i += blockDim.x)
      a.seq_len[a.layer * g.n_seqs + a.seq_begin + i] += a.n_tokens;
  }
}

__global__ void clear_kernel(int32_t* seq_len, uint32_t* cursor, int layer, int n_seqs,
                             int n_heads, int seq_begin, int seq_count) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < seq_count) seq_len[layer * n_seqs + seq_begin + i] = 0;
  if (i < seq_count * n_heads)
    cursor[((size_t)layer * n_seqs + seq_begin) * n_heads + i] = 0u;
}

constexpr int VALUE_ENCODER_DEFAULT = 1;
int g_value_encoder = VALUE_ENCODER_DEFAULT;  // 0: rotation on mma.sync; 1: on tcgen05.mma

template <int DT>
int launch_encode_t(const EncodeArgs& a, int sm_count, int device, cudaStream_t st, int* launches) {
  const tq_geom& g = a.g;
  if (a.max_new_blocks > 0) {
    dim3 grid(a.max_new_blocks, g.n_kv_heads, a.seq_count);
    if (g.key_mode == TQ_KEYS_POLAR) {
      // (the keys go through the value encoder, below)
    } else if (DT == TQ_F32) {
      encode_keys_kernel<DT, false><<<grid, TQ_D, 0, st>>>(a);  // one thread per channel
    } else {
      const int stage_bytes = g.block_tokens * TQ_D * elem_size(DT);
      static bool keys_attr_set[16] = {};
      if (!keys_attr_set[device & 15]) {
        TQ_CUDA(cudaFuncSetAttribute(encode_keys_kernel<DT, true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 256 * TQ_D * 2));
        keys_attr_set[device & 15] = true;
      }
      encode_keys_kernel<DT, true><<<grid, 2 * TQ_D, stage_bytes, st>>>(a);
    }
    int groups = g.block_tokens_pad / TQ_GROUP_TOK;
    long total = (long)a.seq_count * g.n_kv_heads * a.max_new_blocks * groups;
    // one wave: two CTAs per SM, each working on two 16-token groups at a time
    int ctas = (int)std::min<long>((total + ENCV_HALVES - 1) / ENCV_HALVES, (long)sm_count * 2);
    static bool attr_set[16] = {};  // per device: the attribute belongs to the device's context
    if (!attr_set[device & 15]) {
      TQ_CUDA(cudaFuncSetAttribute(encode_values_kernel<DT>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, ENCV_SMEM));
      attr_set[device & 15] = true;
    }
    static bool attr5_set[16] = {};
    const bool tc5 = g_value_encoder == 1;
    if (tc5 && !attr5_set[device & 15]) {
      TQ_CUDA(cudaFuncSetAttribute(encode_values_tc5_kernel<DT, 3>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, ENC5_SMEM));
      TQ_CUDA(cudaFuncSetAttribute(encode_values_tc5_kernel<DT, 4>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, ENC5_SMEM));
      attr5_set[device & 15] = true;
    }
    const int ctas5 = (int)std::min<long>((total + ENC5_PARTS - 1) / ENC5_PARTS, (long)sm_count);
    auto values = [&](const EncodeArgs& av) {
      if (tc5 && g.value_bits == 3)
        encode_values_tc5_kernel<DT, 3><<<ctas5, ENC5_PARTS * TQ_D, ENC5_SMEM, st>>>(av);
      else if (tc5)
        encode_values_tc5_kernel<DT, 4><<<ctas5, ENC5_PARTS * TQ_D, ENC5_SMEM, st>>>(av);
      else
        encode_values_kernel<DT><<<ctas, ENCV_HALVES * TQ_D, ENCV_SMEM, st>>>(av);
    };
    if (g.key_mode == TQ_KEYS_POLAR) {
      EncodeArgs ak = a;
      ak.polar_keys_pass = 1;
      values(ak);
    }
    values(a);
    *launches += 2;
  }
  // (launched so that it may be scheduled while the kernel before it in the stream drains; it
  // waits for that kernel itself)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(std::min(a.n_tokens, g.hot_window), g.n_kv_heads, a.seq_count);
  cfg.blockDim = dim3(TQ_D);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TQ_CUDA(cudaLaunchKernelEx(&cfg, ring_write_kernel<DT>, a));
  *launches += 1;
  return TQ_OK;
}

}  // namespace

extern "C" int32_t tq_set_value_encoder(int32_t kind) {
  TQ_REQUIRE(kind >= -1 && kind <= 1, TQ_ERR_INVALID,
             "value encoder: 0 (mma.sync), 1 (tcgen05) or -1 (the default)");
  g_value_encoder = kind < 0 ? VALUE_ENCODER_DEFAULT : kind;
  return TQ_OK;
}

int tq_launch_encode(tq_ctx* ctx, int layer, int seq_begin, int seq_count, const void* k,
                     const void* v, int n_tokens, int64_t seq_stride, int64_t tok_stride,
                     int64_t head_stride, int max_new_blocks, cudaStream_t st) {
  EncodeArgs a;
  a.g = ctx->g;
  a.pages = (uint8_t*)ctx->b.pages;
  a.hot_k = ctx->b.hot_k;
  a.hot_v = ctx->b.hot_v;
  a.pool_dec = (uint32_t*)ctx->b.pool_dec;
  a.pool_val = (uint16_t*)ctx->b.pool_val;
  a.page_meta = (PageMeta*)ctx->b.page_meta;
  a.seq_len = (int32_t*)((uint8_t*)ctx->b.state + state_len_off(ctx->g));
  a.pool_cursor = (uint32_t*)((uint8_t*)ctx->b.state + state_cursor_off(ctx->g));
  a.status = (int32_t*)((uint8_t*)ctx->b.state + state_status_off(ctx->g));
  a.tables = (const Tables*)ctx->b.tables;
  a.bias_means = ctx->bias_means
                     ? (const float*)((const uint8_t*)ctx->b.tables + align_up(sizeof(Tables), 256))
                     : nullptr;
  a.k = k;
  a.v = v;
  a.layer = layer;
  a.seq_begin = seq_begin;
  a.seq_count = seq_count;
  a.n_tokens = n_tokens;
  a.max_new_blocks = max_new_blocks;
  a.polar_keys_pass = 0;
  a.seq_stride = seq_stride;
  a.tok_stride = tok_stride;
  a.head_stride = head_stride;
  int sm_count = 148;
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, ctx->device);
  int launches = 0;
  switch (ctx->g.kv_dtype) {
    case TQ_F32: launch_encode_t<TQ_F32>(a, sm_count, ctx->device, st, &launches); break;
    case TQ_F16: launch_encode_t<TQ_F16>(a, sm_count, ctx->device, st, &launches); break;
    default: launch_encode_t<TQ_BF16>(a, sm_count, ctx->device, st, &launches); break;
  }
  ctx->last_launches = launches;
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}

int tq_launch_clear(tq_ctx* ctx, int layer, int seq_begin, int seq_count, cudaStream_t st) {
  const tq_geom& g = ctx->g;
  int32_t* seq_len = (int32_t*)((uint8_t*)ctx->b.state + state_len_off(g));
  uint32_t* cursor = (uint32_t*)((uint8_t*)ctx->b.state + state_cursor_off(g));
  int n = seq_count * g.n_kv_heads;
  clear_kernel<<<(n + 127) / 128, 128, 0, st>>>(seq_len, cursor, layer, g.n_seqs, g.n_kv_heads,
                                                seq_begin, seq_count);
  size_t first = unit_index(g, layer, seq_begin, 0) * g.max_blocks;
  TQ_CUDA(cudaMemsetAsync((PageMeta*)ctx->b.page_meta + first, 0,
                          (size_t)n * g.max_blocks * sizeof(PageMeta), st));
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}
