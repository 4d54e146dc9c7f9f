// Dequantised read-back of a token range (the get_keys / get_values getters).  The result
// is bit-identical to the reference decoders: keys are fl(fl(scale * NF4[code]) + mean)
// with outlier positions overwritten by their fp16 values; values are
// (centroid[code] @ Pi) * norm with the rotation accumulated sequentially and unfused.
#include "common.cuh"

namespace {

struct DequantArgs {
  tq_geom g;
  const uint8_t* pages;
  const void* hot_k;
  const void* hot_v;
  const uint32_t* pool_dec;
  const uint16_t* pool_val;
  const PageMeta* page_meta;
  const Tables* tables;
  int layer, seq, start, end, n_total;
  float* k_out;  // [H][end-start][D]
  float* v_out;
  int keys_pass;  // PolarQuant keys: the value kernel reads the key codes and writes k_out
};

TQ_DEV float ld_any(const void* p, size_t i, int dt) {
  if (dt == TQ_F32) return ((const float*)p)[i];
  if (dt == TQ_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// keys + hot tokens of both tensors: grid = (token, head), thread = channel
__global__ void __launch_bounds__(TQ_D) dequant_dense_kernel(DequantArgs a) {
  const tq_geom& g = a.g;
  const int pos = a.start + blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int S = g.block_tokens;
  const int nb = n_cold_blocks(a.n_total, g.hot_window, S);
  const size_t o = ((size_t)head * (a.end - a.start) + blockIdx.x) * TQ_D + d;
  if (pos < nb * S) {
    if (a.k_out == nullptr || g.key_mode == TQ_KEYS_POLAR) return;
    const int blk = pos / S, t = pos % S;
    const uint8_t* page = a.pages + page_offset(g, a.layer, a.seq, head, blk);
    const uint8_t b = page[t * (TQ_D / 2) + (d >> 1)];
    const int code = (d & 1) ? (b >> 4) : (b & 15);
    const float sc = ((const float*)(page + g.scale_off))[d];
    const float mu = ((const float*)(page + g.mean_off))[d];
    // symmetric NF4 stores mean 0, uniform keys are fl(fl(code * scale) + zero): one form
    a.k_out[o] = __fadd_rn(__fmul_rn(sc, a.tables->grid[code]), mu);
  } else {
    const size_t i = hot_offset_elems(g, a.layer, a.seq, head) + (size_t)(pos % g.hot_cap) * TQ_D + d;
    if (a.k_out) a.k_out[o] = ld_any(a.hot_k, i, g.kv_dtype);
    if (a.v_out) a.v_out[o] = ld_any(a.hot_v, i, g.kv_dtype);
  }
}

// outlier overwrite: grid = (block, head), threads stride over the block's side-list
__global__ void dequant_outlier_kernel(DequantArgs a, int blk0) {
  const tq_geom& g = a.g;
  const int blk = blk0 + blockIdx.x, head = blockIdx.y;
  const int S = g.block_tokens;
  const PageMeta pm = a.page_meta[unit_index(g, a.layer, a.seq, head) * g.max_blocks + blk];
  const size_t slab = unit_index(g, a.layer, a.seq, head) * (size_t)g.pool_entries + pm.off;
  for (uint32_t e = threadIdx.x; e < pm.cnt; e += blockDim.x) {
    const uint32_t w = a.pool_dec[slab + e];
    const int col = (w >> 16) & 255, tok = w >> 24;
    const int pos = blk * S + tok;
    if (pos < a.start || pos >= a.end) continue;
    const size_t o = ((size_t)head * (a.end - a.start) + (pos - a.start)) * TQ_D + col;
    a.k_out[o] = __half2float(__ushort_as_half(a.pool_val[slab + e]));
  }
}

// cold values: grid = (16-token group index over the covered blocks, head), thread = output
// channel; same sequential, unfused rotation as the encoder, with Pi instead of Pi^T
__global__ void __launch_bounds__(TQ_D) dequant_values_kernel(DequantArgs a, int blk0) {
  const tq_geom& g = a.g;
  const int groups = g.block_tokens_pad / TQ_GROUP_TOK;
  const int blk = blk0 + blockIdx.x / groups, gq = blockIdx.x % groups;
  const int head = blockIdx.y, e = threadIdx.x;
  const int S = g.block_tokens, vb = g.value_bits;
  const uint8_t* page = a.pages + page_offset(g, a.layer, a.seq, head, blk);
  const uint8_t* grp = page + (a.keys_pass ? 0 : g.v_off) + (size_t)gq * v_group_bytes(vb);
  __shared__ __align__(16) float us[TQ_D][TQ_GROUP_TOK];
  __shared__ float cent[16];
  if (e < 16) cent[e] = a.tables->centroids[e];
  __syncthreads();
#pragma unroll 4
  for (int t = 0; t < TQ_GROUP_TOK; ++t) us[e][t] = cent[v_get_code(grp, vb, t, e)];
  __syncthreads();
  float acc[TQ_GROUP_TOK];
  {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float4 u = *(const float4*)&us[0][4 * q];
      float p0 = a.tables->pi[e];
      acc[4 * q + 0] = __fmul_rn(u.x, p0);
      acc[4 * q + 1] = __fmul_rn(u.y, p0);
      acc[4 * q + 2] = __fmul_rn(u.z, p0);
      acc[4 * q + 3] = __fmul_rn(u.w, p0);
    }
    for (int dd = 1; dd < TQ_D; ++dd) {
      const float pv = a.tables->pi[dd * TQ_D + e];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float4 u = *(const float4*)&us[dd][4 * q];
        acc[4 * q + 0] = __fadd_rn(acc[4 * q + 0], __fmul_rn(u.x, pv));
        acc[4 * q + 1] = __fadd_rn(acc[4 * q + 1], __fmul_rn(u.y, pv));
        acc[4 * q + 2] = __fadd_rn(acc[4 * q + 2], __fmul_rn(u.z, pv));
        acc[4 * q + 3] = __fadd_rn(acc[4 * q + 3], __fmul_rn(u.w, pv));
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TQ_GROUP_TOK; ++t) {
    const int tt = gq * TQ_GROUP_TOK + t;
    const int pos = blk * S + tt;
    if (tt < S && pos >= a.start && pos < a.end) {
      const float nrm = ((const float*)(page + (a.keys_pass ? g.scale_off : g.norm_off)))[tt];
      (a.keys_pass ? a.k_out : a.v_out)[((size_t)head * (a.end - a.start) + (pos - a.start)) * TQ_D + e] =
          __fmul_rn(acc[t], nrm);
    }
  }
}

}  // namespace

int tq_launch_dequant(tq_ctx* ctx, int layer, int seq, int start, int end, float* k_out,
                      float* v_out, cudaStream_t st) {
  const tq_geom& g = ctx->g;
  DequantArgs a;
  a.g = g;
  a.pages = (const uint8_t*)ctx->b.pages;
  a.hot_k = ctx->b.hot_k;
  a.hot_v = ctx->b.hot_v;
  a.pool_dec = (const uint32_t*)ctx->b.pool_dec;
  a.pool_val = (const uint16_t*)ctx->b.pool_val;
  a.page_meta = (const PageMeta*)ctx->b.page_meta;
  a.tables = (const Tables*)ctx->b.tables;
  a.layer = layer;
  a.seq = seq;
  a.start = start;
  a.end = end;
  a.n_total = ctx->len[(size_t)layer * g.n_seqs + seq];
  a.k_out = k_out;
  a.v_out = v_out;
  a.keys_pass = 0;
  const int S = g.block_tokens;
  const int nb = n_cold_blocks(a.n_total, g.hot_window, S);
  dim3 grid(end - start, g.n_kv_heads);
  dequant_dense_kernel<<<grid, TQ_D, 0, st>>>(a);
  const int cold_end = std::min(end, nb * S);
  if (start < cold_end) {
    const int blk0 = start / S, blk1 = (cold_end - 1) / S;
    if (k_out != nullptr && g.outlier_k > 0) {
      dim3 go(blk1 - blk0 + 1, g.n_kv_heads);
      dequant_outlier_kernel<<<go, 256, 0, st>>>(a, blk0);
    }
    const int groups = g.block_tokens_pad / TQ_GROUP_TOK;
    dim3 gv((blk1 - blk0 + 1) * groups, g.n_kv_heads);
    if (v_out != nullptr) dequant_values_kernel<<<gv, TQ_D, 0, st>>>(a, blk0);
    if (k_out != nullptr && g.key_mode == TQ_KEYS_POLAR) {
      // PolarQuant keys: TurboQuantKV.decompress on the key codes (core.py:619-654)
      DequantArgs ak = a;
      ak.keys_pass = 1;
      dequant_values_kernel<<<gv, TQ_D, 0, st>>>(ak, blk0);
    }
  }
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}
