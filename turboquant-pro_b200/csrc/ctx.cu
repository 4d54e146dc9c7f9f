// Host side of the C ABI: geometry, region sizes, context lifetime, append bookkeeping,
// export to the reference's container layout, statistics.  No kernels live here.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.cuh"

// the NF4 levels (float32), as the reference's table holds them
static const float nf4[16] = {-1.0f,
    -0.6961928009986877f,
    -0.5250730514526367f,
    -0.39491748809814453f,
    -0.28444138169288635f,
    -0.18477343022823334f,
    -0.09105003625154495f,
    0.0f,
    0.07958029955625534f,
    0.16093020141124725f,
    0.24611230194568634f,
    0.33791524171829224f,
    0.44070982933044434f,
    0.5626170039176941f,
    0.7229568362236023f,
    1.0f};

static thread_local std::string g_last_error;

void tq_set_error(const std::string& msg) { g_last_error = msg; }

int tq_cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return TQ_ERR_CUDA;
}

cudaEvent_t tq_prof_event(tq_ctx* ctx, int i) {
  if (!ctx->prof_on || ctx->prof_n >= TQ_PROF_MAX) return nullptr;
  size_t idx = (size_t)ctx->prof_n * 3 + i;
  while (ctx->prof_ev.size() <= idx) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    ctx->prof_ev.push_back(e);
  }
  return ctx->prof_ev[idx];
}

void tq_prof_commit(tq_ctx* ctx) {
  if (ctx->prof_on && ctx->prof_n < TQ_PROF_MAX) ctx->prof_n++;
}

static bool good_ctx(const tq_ctx* c, int layer) {
  return c != nullptr && layer >= 0 && layer < c->g.n_layers;
}

struct tq_xchg;
int tq_launch_decode_exchange(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                              int block_end, int with_hot, float* out, const tq_xchg* xchg,
                              int phases, cudaStream_t st, bool* handled);

extern "C" {

int32_t tq_version(void) { return TQ_VERSION; }

const char* tq_last_error(void) { return g_last_error.c_str(); }

int32_t tq_geom_finish(tq_geom* g) {
  TQ_REQUIRE(g != nullptr, TQ_ERR_INVALID, "geometry is null");
  TQ_REQUIRE(g->n_layers >= 1 && g->n_seqs >= 1 && g->n_kv_heads >= 1, TQ_ERR_INVALID,
             "n_layers, n_seqs and n_kv_heads must be positive");
  TQ_REQUIRE(g->n_q_heads >= g->n_kv_heads && g->n_q_heads % g->n_kv_heads == 0, TQ_ERR_INVALID,
             "n_q_heads must be a positive multiple of n_kv_heads");
  TQ_REQUIRE(g->head_dim == TQ_D, TQ_ERR_UNSUPPORTED, "only head_dim == 128 is implemented");
  TQ_REQUIRE(g->key_mode >= TQ_KEYS_NF4_ASYM && g->key_mode <= TQ_KEYS_POLAR, TQ_ERR_INVALID,
             "key_mode must be one of TQ_KEYS_*");
  TQ_REQUIRE(g->value_bits == 3 || g->value_bits == 4, TQ_ERR_UNSUPPORTED,
             "value_bits must be 3 or 4");
  if (g->key_mode == TQ_KEYS_POLAR) {
    TQ_REQUIRE(g->key_bits == g->value_bits, TQ_ERR_UNSUPPORTED,
               "PolarQuant keys: key_bits must equal value_bits");
    TQ_REQUIRE(g->outlier_frac == 0.0, TQ_ERR_INVALID, "PolarQuant keys keep no outliers");
  } else {
    TQ_REQUIRE(g->key_bits == 4, TQ_ERR_UNSUPPORTED, "per-channel keys: key_bits must be 4");
  }
  TQ_REQUIRE(g->hot_window >= 2 && g->hot_window <= 512, TQ_ERR_UNSUPPORTED,
             "hot_window must be in [2, 512]");
  TQ_REQUIRE(g->kv_dtype == TQ_F32 || g->kv_dtype == TQ_F16 || g->kv_dtype == TQ_BF16,
             TQ_ERR_INVALID, "kv_dtype must be TQ_F32, TQ_F16 or TQ_BF16");
  TQ_REQUIRE(g->max_tokens_per_seq >= 1, TQ_ERR_INVALID, "max_tokens_per_seq must be positive");
  TQ_REQUIRE(g->outlier_frac >= 0.0 && g->outlier_frac < 1.0, TQ_ERR_INVALID,
             "outlier_frac must be in [0, 1)");
  g->group = g->n_q_heads / g->n_kv_heads;
  TQ_REQUIRE(g->group <= TQ_MAX_G, TQ_ERR_UNSUPPORTED, "GQA group larger than 16");
  g->block_tokens = (g->hot_window + 1) / 2;
  g->block_tokens_pad = (int)align_up(g->block_tokens, TQ_GROUP_TOK);
  g->hot_cap = (int)align_up(g->hot_window + 1, g->block_tokens);
  g->max_blocks =
      std::max(1, n_cold_blocks(g->max_tokens_per_seq, g->hot_window, g->block_tokens));
  if (g->outlier_frac > 0.0) {
    // max(1, round(S * frac)) with round-half-to-even, as Python's round()
    double r = std::nearbyint((double)g->block_tokens * g->outlier_frac);
    g->outlier_k = std::max(1, (int)r);
    TQ_REQUIRE(g->outlier_k <= TQ_MAX_K_OUT, TQ_ERR_UNSUPPORTED,
               "more than 32 outliers per channel and block");
  } else {
    g->outlier_k = 0;
  }
  g->k_bytes = g->block_tokens_pad * (TQ_D / 2);
  g->v_bytes = g->block_tokens_pad / TQ_GROUP_TOK * v_group_bytes(g->value_bits);
  g->v_off = g->k_bytes;
  g->norm_off = g->v_off + g->v_bytes;
  g->scale_off = g->norm_off + g->block_tokens_pad * 4;
  g->mean_off = g->scale_off + TQ_D * 4;
  g->hdr_off = (int)align_up(g->mean_off + TQ_D * 4, 128);
  g->ent_off = g->hdr_off + TQ_ELL_OFF;
  g->page_bytes = (int)align_up(g->hdr_off + TQ_TAIL_BYTES, 128);
  if (g->outlier_k > 0) {
    int64_t nominal = (int64_t)g->max_blocks * g->outlier_k * TQ_D;
    int64_t cap = nominal + nominal / 4 + 4096;
    TQ_REQUIRE(cap < (1ll << 30), TQ_ERR_UNSUPPORTED, "outlier pool too large");
    g->pool_entries = (int)align_up((size_t)cap, 64);
  } else {
    g->pool_entries = 0;
  }
  g->max_splits = 64;
  g->reserved_ = 0;
  return TQ_OK;
}

int32_t tq_ctx_sizes(const tq_geom* g, tq_sizes* out) {
  TQ_REQUIRE(g != nullptr && out != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(g->page_bytes > 0, TQ_ERR_INVALID, "call tq_geom_finish first");
  size_t units = (size_t)g->n_layers * g->n_seqs * g->n_kv_heads;
  out->pages = align_up(units * g->max_blocks * (size_t)g->page_bytes, 256);
  size_t hot = units * g->hot_cap * (size_t)TQ_D * elem_size(g->kv_dtype);
  out->hot_k = align_up(hot, 256);
  out->hot_v = align_up(hot, 256);
  out->pool_dec = align_up(std::max<size_t>(units * (size_t)g->pool_entries * 4, 256), 256);
  out->pool_val = align_up(std::max<size_t>(units * (size_t)g->pool_entries * 2, 256), 256);
  out->page_meta = align_up(units * g->max_blocks * sizeof(PageMeta), 256);
  out->state = align_up(state_bytes(*g), 256);
  // the Tables struct, then room for given key zero-points [max_blocks][H][D] (float32)
  out->tables = align_up(sizeof(Tables), 256) +
                align_up((size_t)g->max_blocks * g->n_kv_heads * TQ_D * sizeof(float), 256);
  size_t layer_units = (size_t)g->n_seqs * g->n_kv_heads;
  size_t generic = layer_units * g->max_splits * g->group * TQ_PART_STRIDE * sizeof(float);
  out->scratch = align_up(std::max(generic, tq_mma_scratch_bytes(*g, layer_units)), 256);
  return TQ_OK;
}

int32_t tq_ctx_create(const tq_geom* g, const tq_buffers* bufs, int32_t device, const float* pi,
                      const float* pi_t, const float* centroids, const float* boundaries,
                      void* stream, tq_ctx** out) {
  TQ_REQUIRE(g && bufs && pi && pi_t && centroids && boundaries && out, TQ_ERR_INVALID,
             "null argument");
  TQ_REQUIRE(g->page_bytes > 0, TQ_ERR_INVALID, "call tq_geom_finish first");
  const void* ptrs[] = {bufs->pages,     bufs->hot_k, bufs->hot_v,  bufs->pool_dec, bufs->pool_val,
                        bufs->page_meta, bufs->state, bufs->tables, bufs->scratch};
  for (const void* p : ptrs)
    TQ_REQUIRE(p != nullptr && ((uintptr_t)p & 255) == 0, TQ_ERR_INVALID,
               "every region must be a non-null, 256-byte aligned device pointer");
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    tq_set_error("no CUDA device");
    return TQ_ERR_NO_DEVICE;
  }
  TQ_REQUIRE(device >= 0 && device < n_dev, TQ_ERR_INVALID, "device ordinal out of range");
  TQ_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  TQ_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    tq_set_error("this library is built for sm_100a (B200) only");
    return TQ_ERR_NO_DEVICE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  Tables* t = new Tables();
  std::memcpy(t->pi, pi, sizeof(t->pi));
  std::memcpy(t->pi_t, pi_t, sizeof(t->pi_t));
  int nc = 1 << g->value_bits;
  for (int i = 0; i < 16; ++i) {
    t->centroids[i] = i < nc ? centroids[i] : 0.0f;
    t->boundaries[i] = i < nc - 1 ? boundaries[i] : INFINITY;
  }
  for (int i = 0; i < 16; ++i) t->grid[i] = g->key_mode == TQ_KEYS_UNIFORM ? (float)i : nf4[i];
  std::memset(t->mean_mask, 1, sizeof(t->mean_mask));
  cudaError_t e = cudaMemcpyAsync(bufs->tables, t, sizeof(Tables), cudaMemcpyHostToDevice, st);
  // The hot rings start zeroed: the decode kernel multiplies ring rows past the end of a
  // window by probability 0, which needs them finite.
  tq_sizes sz;
  if (e == cudaSuccess && tq_ctx_sizes(g, &sz) == TQ_OK) {
    e = cudaMemsetAsync(bufs->hot_k, 0, sz.hot_k, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(bufs->hot_v, 0, sz.hot_v, st);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    delete t;
    return tq_cuda_fail(e, "uploading tables");
  }
  tq_ctx* c = new tq_ctx();
  c->g = *g;
  c->b = *bufs;
  c->device = device;
  c->len.assign((size_t)g->n_layers * g->n_seqs, 0);
  c->last_launches = 0;
  std::memcpy(c->h_centroids, t->centroids, sizeof(c->h_centroids));
  std::memcpy(c->h_boundaries, t->boundaries, sizeof(c->h_boundaries));
  delete t;
  *out = c;
  return TQ_OK;
}

int32_t tq_ctx_destroy(tq_ctx* ctx) {
  if (ctx != nullptr)
    for (cudaEvent_t e : ctx->prof_ev) cudaEventDestroy(e);
  delete ctx;
  return TQ_OK;
}

int32_t tq_set_key_mean_mask(tq_ctx* ctx, const uint8_t* mask, void* stream) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  TQ_REQUIRE(ctx->g.key_mode == TQ_KEYS_NF4_ASYM, TQ_ERR_INVALID,
             "a mean mask applies to asymmetric NF4 keys only");
  uint8_t m[TQ_D];
  int n = 0;
  for (int d = 0; d < TQ_D; ++d) {
    m[d] = (mask == nullptr || mask[d] != 0) ? 1 : 0;
    n += m[d];
  }
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  TQ_CUDA(cudaMemcpyAsync((uint8_t*)ctx->b.tables + offsetof(Tables, mean_mask), m, TQ_D,
                          cudaMemcpyHostToDevice, st));
  TQ_CUDA(cudaStreamSynchronize(st));  // `m` lives on this stack frame
  ctx->mean_channels = n;
  return TQ_OK;
}

int32_t tq_set_key_bias_means(tq_ctx* ctx, const float* means, void* stream) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  TQ_REQUIRE(ctx->g.key_mode == TQ_KEYS_NF4_ASYM, TQ_ERR_INVALID,
             "given zero-points apply to asymmetric NF4 keys only");
  if (means == nullptr) {
    ctx->bias_means = false;
    return TQ_OK;
  }
  const tq_geom& g = ctx->g;
  const size_t bytes = (size_t)g.max_blocks * g.n_kv_heads * TQ_D * sizeof(float);
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  TQ_CUDA(cudaMemcpyAsync((uint8_t*)ctx->b.tables + align_up(sizeof(Tables), 256), means, bytes,
                          cudaMemcpyHostToDevice, st));
  TQ_CUDA(cudaStreamSynchronize(st));  // the caller's buffer may go away after the call
  ctx->bias_means = true;
  return TQ_OK;
}

int32_t tq_set_kernel(tq_ctx* ctx, int32_t which) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  TQ_REQUIRE(which == 0 || which == 1, TQ_ERR_INVALID, "which must be 0 (auto) or 1 (general)");
  ctx->force_generic = which == 1;
  return TQ_OK;
}

int32_t tq_last_kernel(const tq_ctx* ctx) { return ctx ? ctx->last_kernel : TQ_KERNEL_NONE; }

int32_t tq_debug_wait(tq_ctx* ctx, int32_t wait_limit, int32_t withhold_tile) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  TQ_REQUIRE(wait_limit >= 0 && withhold_tile >= -1, TQ_ERR_INVALID,
             "wait_limit must be >= 0 and withhold_tile >= -1");
  ctx->wait_limit = wait_limit;
  ctx->withhold_tile = withhold_tile;
  return TQ_OK;
}

int32_t tq_debug_trace(tq_ctx* ctx, int32_t on, uint64_t* stamps, void* stream) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  ctx->trace_on = on != 0;
  if (stamps != nullptr) {
    TQ_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    TQ_CUDA(cudaMemcpyAsync(stamps, (const uint8_t*)ctx->b.scratch, TQ_MMA_TRACE_BYTES,
                            cudaMemcpyDeviceToHost, st));
    TQ_CUDA(cudaStreamSynchronize(st));
  }
  return TQ_OK;
}

int32_t tq_profile_enable(tq_ctx* ctx, int32_t on) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  ctx->prof_on = on != 0;
  return TQ_OK;
}

int32_t tq_profile_read(tq_ctx* ctx, double* attn_ms, double* combine_ms, int32_t* n_calls) {
  TQ_REQUIRE(ctx != nullptr, TQ_ERR_INVALID, "null context");
  double a = 0.0, c = 0.0;
  for (int i = 0; i < ctx->prof_n; ++i) {
    cudaEvent_t* e = &ctx->prof_ev[(size_t)i * 3];
    TQ_CUDA(cudaEventSynchronize(e[2]));
    float t0 = 0.f, t1 = 0.f;
    TQ_CUDA(cudaEventElapsedTime(&t0, e[0], e[1]));
    TQ_CUDA(cudaEventElapsedTime(&t1, e[1], e[2]));
    a += t0;
    c += t1;
  }
  if (attn_ms) *attn_ms = a;
  if (combine_ms) *combine_ms = c;
  if (n_calls) *n_calls = ctx->prof_n;
  ctx->prof_n = 0;
  return TQ_OK;
}

int32_t tq_append(tq_ctx* ctx, int32_t layer, int32_t seq_begin, int32_t seq_count,
                  const void* k, const void* v, int32_t n_tokens, int64_t seq_stride,
                  int64_t tok_stride, int64_t head_stride, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq_begin >= 0 && seq_count >= 1 && seq_begin + seq_count <= g.n_seqs,
             TQ_ERR_INVALID, "sequence range out of bounds");
  TQ_REQUIRE(n_tokens >= 0, TQ_ERR_INVALID, "n_tokens must be non-negative");
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(k != nullptr && v != nullptr, TQ_ERR_INVALID, "k and v must be device pointers");
  int max_new = 0;
  for (int s = seq_begin; s < seq_begin + seq_count; ++s) {
    int n0 = ctx->len[(size_t)layer * g.n_seqs + s];
    TQ_REQUIRE((int64_t)n0 + n_tokens <= g.max_tokens_per_seq, TQ_ERR_CAPACITY,
               "append exceeds max_tokens_per_seq");
    int nb0 = n_cold_blocks(n0, g.hot_window, g.block_tokens);
    int nb1 = n_cold_blocks(n0 + n_tokens, g.hot_window, g.block_tokens);
    max_new = std::max(max_new, nb1 - nb0);
  }
  TQ_CUDA(cudaSetDevice(ctx->device));
  int rc = tq_launch_encode(ctx, layer, seq_begin, seq_count, k, v, n_tokens, seq_stride,
                            tok_stride, head_stride, max_new, (cudaStream_t)stream);
  if (rc != TQ_OK) return rc;
  for (int s = seq_begin; s < seq_begin + seq_count; ++s)
    ctx->len[(size_t)layer * g.n_seqs + s] += n_tokens;
  return TQ_OK;
}

int32_t tq_decode(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype, float* out,
                  void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(q != nullptr && out != nullptr, TQ_ERR_INVALID, "q and out must be device pointers");
  TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16 || q_dtype == TQ_BF16, TQ_ERR_INVALID,
             "bad q_dtype");
  TQ_CUDA(cudaSetDevice(ctx->device));
  ctx->last_q_dtype = q_dtype;
  return tq_launch_decode(ctx, layer, q, q_dtype, 0, -1, 1, out, nullptr, (cudaStream_t)stream);
}

int32_t tq_decode_partial(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype,
                          int32_t block_begin, int32_t block_end, int32_t with_hot, float* mlo,
                          void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(q != nullptr && mlo != nullptr, TQ_ERR_INVALID, "q and mlo must be device pointers");
  TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16 || q_dtype == TQ_BF16, TQ_ERR_INVALID,
             "bad q_dtype");
  TQ_REQUIRE(block_begin >= 0 && block_end >= block_begin, TQ_ERR_INVALID, "bad block range");
  TQ_CUDA(cudaSetDevice(ctx->device));
  ctx->last_q_dtype = q_dtype;
  return tq_launch_decode(ctx, layer, q, q_dtype, block_begin, block_end, with_hot ? 1 : 0,
                          nullptr, mlo, (cudaStream_t)stream);
}

int32_t tq_decode_exchange(tq_ctx* ctx, int32_t layer, const void* q, int32_t q_dtype,
                           int32_t block_begin, int32_t block_end, int32_t with_hot, tq_xchg* xchg,
                           float* out, int32_t phases, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(q != nullptr && xchg != nullptr, TQ_ERR_INVALID, "q and xchg must not be null");
  TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16 || q_dtype == TQ_BF16, TQ_ERR_INVALID,
             "bad q_dtype");
  TQ_REQUIRE(block_begin >= 0 && block_end >= block_begin, TQ_ERR_INVALID, "bad block range");
  TQ_REQUIRE(phases == 1 || phases == 3, TQ_ERR_INVALID,
             "phases: 3 publish, wait and merge; 1 publish only (then tq_xchg_gather_merge with 2)");
  TQ_REQUIRE(out != nullptr || phases == 1, TQ_ERR_INVALID, "out must be a device pointer");
  TQ_CUDA(cudaSetDevice(ctx->device));
  ctx->last_q_dtype = q_dtype;
  bool handled = false;
  int rc = tq_launch_decode_exchange(ctx, layer, q, q_dtype, block_begin, block_end,
                                     with_hot ? 1 : 0, out, xchg, phases, (cudaStream_t)stream,
                                     &handled);
  if (rc != TQ_OK) return rc;
  TQ_REQUIRE(handled, TQ_ERR_UNSUPPORTED,
             "this geometry has no fused exchange: use tq_decode_partial + tq_xchg_gather_merge");
  return TQ_OK;
}

int32_t tq_lse_combine(const float* mlo, int32_t n_parts, int32_t n_rows, int32_t head_dim,
                       float* out, void* stream) {
  TQ_REQUIRE(mlo != nullptr && out != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_REQUIRE(n_parts >= 1 && n_rows >= 1, TQ_ERR_INVALID, "n_parts and n_rows must be positive");
  TQ_REQUIRE(head_dim == TQ_D, TQ_ERR_UNSUPPORTED, "only head_dim == 128 is implemented");
  return tq_launch_lse_combine(mlo, n_parts, n_rows, head_dim, out, (cudaStream_t)stream);
}

int32_t tq_dequant_range(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t start, int32_t end,
                         float* k_out, float* v_out, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(seq >= 0 && seq < ctx->g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int n = ctx->len[(size_t)layer * ctx->g.n_seqs + seq];
  TQ_REQUIRE(start >= 0 && end >= start && end <= n, TQ_ERR_INVALID, "token range out of bounds");
  if (end == start || (k_out == nullptr && v_out == nullptr)) return TQ_OK;
  TQ_CUDA(cudaSetDevice(ctx->device));
  return tq_launch_dequant(ctx, layer, seq, start, end, k_out, v_out, (cudaStream_t)stream);
}

int32_t tq_seq_lengths(const tq_ctx* ctx, int32_t layer, int32_t seq, int32_t* total,
                       int32_t* cold, int32_t* hot) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(seq >= 0 && seq < ctx->g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int n = ctx->len[(size_t)layer * ctx->g.n_seqs + seq];
  int nb = n_cold_blocks(n, ctx->g.hot_window, ctx->g.block_tokens);
  if (total) *total = n;
  if (cold) *cold = nb * ctx->g.block_tokens;
  if (hot) *hot = n - nb * ctx->g.block_tokens;
  return TQ_OK;
}

static uint8_t rev4(uint8_t c) {
  return (uint8_t)(((c & 1) << 3) | ((c & 2) << 1) | ((c & 4) >> 1) | ((c & 8) >> 3));
}

int32_t tq_export_block(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t block,
                        uint8_t* key_indices, float* nf4_scale, float* nf4_mean,
                        int32_t* outlier_idx, uint16_t* outlier_val, int32_t outlier_cap,
                        int32_t* n_outliers, uint8_t* value_indices, float* value_norms,
                        void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq >= 0 && seq < g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int n = ctx->len[(size_t)layer * g.n_seqs + seq];
  int nb = n_cold_blocks(n, g.hot_window, g.block_tokens);
  TQ_REQUIRE(block >= 0 && block < nb, TQ_ERR_INVALID, "block index out of range");
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  const int H = g.n_kv_heads, S = g.block_tokens, D = TQ_D;
  std::vector<uint8_t> page((size_t)H * g.page_bytes);
  std::vector<PageMeta> meta(H);
  for (int h = 0; h < H; ++h) {
    TQ_CUDA(cudaMemcpyAsync(page.data() + (size_t)h * g.page_bytes,
                            (const uint8_t*)ctx->b.pages + page_offset(g, layer, seq, h, block),
                            g.page_bytes, cudaMemcpyDeviceToHost, st));
    size_t mi = unit_index(g, layer, seq, h) * g.max_blocks + block;
    TQ_CUDA(cudaMemcpyAsync(&meta[h], (const PageMeta*)ctx->b.page_meta + mi, sizeof(PageMeta),
                            cudaMemcpyDeviceToHost, st));
  }
  TQ_CUDA(cudaStreamSynchronize(st));
  int total_out = 0;
  for (int h = 0; h < H; ++h) total_out += (int)meta[h].cnt;
  std::vector<uint32_t> dec(std::max(total_out, 1));
  std::vector<uint16_t> val(std::max(total_out, 1));
  {
    int at = 0;
    for (int h = 0; h < H; ++h) {
      if (meta[h].cnt == 0) continue;
      size_t slab = unit_index(g, layer, seq, h) * (size_t)g.pool_entries + meta[h].off;
      TQ_CUDA(cudaMemcpyAsync(dec.data() + at, (const uint32_t*)ctx->b.pool_dec + slab,
                              meta[h].cnt * 4, cudaMemcpyDeviceToHost, st));
      TQ_CUDA(cudaMemcpyAsync(val.data() + at, (const uint16_t*)ctx->b.pool_val + slab,
                              meta[h].cnt * 2, cudaMemcpyDeviceToHost, st));
      at += (int)meta[h].cnt;
    }
    TQ_CUDA(cudaStreamSynchronize(st));
  }
  // value-layout codes of one head's page -> the reference's LSB-first bit stream
  auto pack_stream = [&](const uint8_t* vpg, uint8_t* out, int h, int bits) {
    size_t base_bits = (size_t)h * S * D * bits;  // multiple of 8 because D is
    uint8_t* dst = out + base_bits / 8;
    std::memset(dst, 0, (size_t)S * D * bits / 8);
    for (int s = 0; s < S; ++s) {
      const uint8_t* grp = vpg + (size_t)(s / TQ_GROUP_TOK) * v_group_bytes(bits);
      for (int d = 0; d < D; ++d) {
        int code = v_get_code(grp, bits, s % TQ_GROUP_TOK, d);
        size_t bit = ((size_t)s * D + d) * bits;
        dst[bit >> 3] |= (uint8_t)(code << (bit & 7));
        if ((bit & 7) + bits > 8) dst[(bit >> 3) + 1] |= (uint8_t)(code >> (8 - (bit & 7)));
      }
    }
  };
  const bool polar = g.key_mode == TQ_KEYS_POLAR;
  for (int h = 0; h < H; ++h) {
    const uint8_t* pg = page.data() + (size_t)h * g.page_bytes;
    if (polar) {
      // PolarQuant keys: the key container is a CompressedKV (codes + norms, core.py:596-607)
      if (key_indices) pack_stream(pg, key_indices, h, g.key_bits);
      if (nf4_scale) std::memcpy(nf4_scale + (size_t)h * S, pg + g.scale_off, S * 4);
    } else if (key_indices) {
      for (int s = 0; s < S; ++s)
        for (int j = 0; j < D / 2; ++j) {
          uint8_t b = pg[s * (D / 2) + j];
          key_indices[((size_t)h * S + s) * (D / 2) + j] =
              (uint8_t)((rev4(b & 15) << 4) | rev4(b >> 4));
        }
    }
    if (nf4_scale && !polar) std::memcpy(nf4_scale + (size_t)h * D, pg + g.scale_off, D * 4);
    if (nf4_mean && !polar) std::memcpy(nf4_mean + (size_t)h * D, pg + g.mean_off, D * 4);
    if (value_norms) std::memcpy(value_norms + (size_t)h * S, pg + g.norm_off, S * 4);
    if (value_indices) pack_stream(pg + g.v_off, value_indices, h, g.value_bits);
  }
  if (n_outliers) *n_outliers = total_out;
  if (outlier_idx || outlier_val) {
    TQ_REQUIRE(total_out <= outlier_cap, TQ_ERR_CAPACITY, "outlier_cap too small");
    std::vector<std::pair<int32_t, uint16_t>> ent;
    ent.reserve(total_out);
    int at = 0;
    for (int h = 0; h < H; ++h)
      for (uint32_t e = 0; e < meta[h].cnt; ++e, ++at) {
        uint32_t w = dec[at];
        int col = (w >> 16) & 255, tok = (w >> 24) & 255;
        ent.emplace_back((int32_t)(((size_t)h * S + tok) * D + col), val[at]);
      }
    std::sort(ent.begin(), ent.end(),
              [](const std::pair<int32_t, uint16_t>& a, const std::pair<int32_t, uint16_t>& b) {
                return a.first < b.first;
              });
    for (int i = 0; i < total_out; ++i) {
      if (outlier_idx) outlier_idx[i] = ent[i].first;
      if (outlier_val) outlier_val[i] = ent[i].second;
    }
  }
  return TQ_OK;
}

// Writes code (t, d) of a 16-token group into its records (the inverse of v_get_code; the
// group's bytes start zeroed).
static void v_put_code(uint8_t* grp, int bits, int t, int d, int code) {
  const int l = v_lane(t, d), p = v_pair(t, d), odd = t & 1;
  if (bits == 4) {
    grp[v_record_byte_off(4, l, p)] |= (uint8_t)(code << (odd * 4));
    return;
  }
  const int bit = 6 * p + 3 * odd;
  const int w = code << (bit & 7);
  grp[v_record_byte_off(3, l, bit >> 3)] |= (uint8_t)w;
  if ((w >> 8) != 0) grp[v_record_byte_off(3, l, (bit >> 3) + 1)] |= (uint8_t)(w >> 8);
}

int32_t tq_import_block(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t block,
                        const uint8_t* key_indices, const float* key_scale, const float* key_mean,
                        const int32_t* outlier_idx, const uint16_t* outlier_val,
                        int32_t n_outliers, const uint8_t* value_indices,
                        const float* value_norms, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  TQ_REQUIRE(ctx->g.key_mode != TQ_KEYS_POLAR, TQ_ERR_UNSUPPORTED,
             "import of PolarQuant-key blocks is not implemented");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq >= 0 && seq < g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  TQ_REQUIRE(ctx->len[(size_t)layer * g.n_seqs + seq] == 0, TQ_ERR_INVALID,
             "blocks are imported into a cleared cache, before tq_restore_hot sets its length");
  TQ_REQUIRE(block >= 0 && block < g.max_blocks, TQ_ERR_CAPACITY, "block index out of range");
  TQ_REQUIRE(key_indices && key_scale && key_mean && value_indices && value_norms,
             TQ_ERR_INVALID, "null container array");
  TQ_REQUIRE(n_outliers >= 0 && (n_outliers == 0 || (outlier_idx && outlier_val)),
             TQ_ERR_INVALID, "outlier arrays missing");
  const int H = g.n_kv_heads, S = g.block_tokens, D = TQ_D, vb = g.value_bits;
  for (int i = 0; i < n_outliers; ++i) {
    TQ_REQUIRE(outlier_idx[i] >= 0 && outlier_idx[i] < H * S * D &&
                   (i == 0 || outlier_idx[i] > outlier_idx[i - 1]),
               TQ_ERR_INVALID, "outlier indices must ascend inside the (H, S, D) block");
  }
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* cursor_d = (uint32_t*)((uint8_t*)ctx->b.state + state_cursor_off(g)) +
                       unit_index(g, layer, seq, 0);
  std::vector<uint32_t> cursor(H);
  TQ_CUDA(cudaMemcpyAsync(cursor.data(), cursor_d, H * 4, cudaMemcpyDeviceToHost, st));
  TQ_CUDA(cudaStreamSynchronize(st));

  std::vector<uint8_t> pages((size_t)H * g.page_bytes, 0);
  std::vector<PageMeta> meta(H);
  std::vector<std::vector<uint32_t>> dec(H);
  std::vector<std::vector<uint16_t>> val(H);
  bool pool_short = false;
  int oi = 0;  // position in the outlier arrays (sorted by head, token, channel)
  for (int h = 0; h < H; ++h) {
    uint8_t* pg = pages.data() + (size_t)h * g.page_bytes;
    // key codes: the container holds bit-reversed nibbles, first channel of a pair on top
    for (int s = 0; s < S; ++s)
      for (int j = 0; j < D / 2; ++j) {
        const uint8_t b = key_indices[((size_t)h * S + s) * (D / 2) + j];
        pg[s * (D / 2) + j] = (uint8_t)(rev4(b >> 4) | (rev4(b & 15) << 4));
      }
    float* scale = (float*)(pg + g.scale_off);
    float* mean = (float*)(pg + g.mean_off);
    std::memcpy(scale, key_scale + (size_t)h * D, D * 4);
    std::memcpy(mean, key_mean + (size_t)h * D, D * 4);
    std::memcpy(pg + g.norm_off, value_norms + (size_t)h * S, S * 4);
    // value codes: LSB-first bit stream over (token, channel) -> tensor-core records
    {
      const uint8_t* src = value_indices + (size_t)h * S * D * vb / 8;
      uint8_t* vpg = pg + g.v_off;
      for (int s = 0; s < S; ++s) {
        uint8_t* grp = vpg + (size_t)(s / TQ_GROUP_TOK) * v_group_bytes(vb);
        for (int d = 0; d < D; ++d) {
          const size_t bit = ((size_t)s * D + d) * vb;
          int w = src[bit >> 3];
          if ((bit & 7) + vb > 8) w |= src[(bit >> 3) + 1] << 8;
          v_put_code(grp, vb, s % TQ_GROUP_TOK, d, (w >> (bit & 7)) & ((1 << vb) - 1));
        }
      }
    }
    // header: the four widest channels (largest scale first, ties to the lower channel) and
    // a second copy of their codes, token by token
    PageHeader* hdr = (PageHeader*)(pg + g.hdr_off);
    {
      int order[TQ_D];
      for (int d = 0; d < D; ++d) order[d] = d;
      std::stable_sort(order, order + D, [&](int x, int y) { return scale[x] > scale[y]; });
      uint16_t* side = (uint16_t*)(pg + g.hdr_off + TQ_SIDE_OFF);
      for (int rk = 0; rk < TQ_WIDE; ++rk) {
        const int d = order[rk];
        hdr->wide[rk] = (uint8_t)d;
        for (int t = 0; t < S; ++t) {
          const int code = (pg[t * (D / 2) + (d >> 1)] >> (4 * (d & 1))) & 15;
          side[t] |= (uint16_t)(code << (4 * rk));
        }
      }
    }
    // outliers of this head, grouped by token: the first TQ_ELL_SLOTS of a token go to its
    // fixed slots, the rest to the page's overflow list; all of them to the pool
    const int first = oi;
    while (oi < n_outliers && outlier_idx[oi] < (h + 1) * S * D) ++oi;
    const int n = oi - first;
    uint16_t* ell_delta = (uint16_t*)(pg + g.hdr_off + TQ_ELL_OFF);
    uint8_t* ell_col = pg + g.hdr_off + TQ_ELL_COL_OFF;
    uint32_t* ovf = (uint32_t*)(pg + g.hdr_off + TQ_OVF_OFF);
    int n_ovf = 0, tok_prev = -1, in_tok = 0;
    uint16_t ovf_start[5] = {0, 0, 0, 0, 0};
    dec[h].resize(n);
    val[h].resize(n);
    for (int i = 0; i < n; ++i) {
      const int flat = outlier_idx[first + i] - h * S * D;
      const int t = flat / D, d = flat % D;
      in_tok = t == tok_prev ? in_tok + 1 : 0;
      tok_prev = t;
      const int code = (pg[t * (D / 2) + (d >> 1)] >> (4 * (d & 1))) & 15;
      const float gl = g.key_mode == TQ_KEYS_UNIFORM ? (float)code : nf4[code];
      volatile float sl = scale[d] * gl;  // rounded to float32 on its own, like the encoder
      volatile float dense = g.key_mode == TQ_KEYS_NF4 ? (float)sl : mean[d] + sl;
      const __half hv = __ushort_as_half(outlier_val[first + i]);
      volatile float diff = __half2float(hv) - dense;
      const uint16_t delta = __half_as_ushort(__float2half_rn(diff));
      const uint32_t ent = (uint32_t)delta | ((uint32_t)d << 16) | ((uint32_t)t << 24);
      dec[h][i] = ent;
      val[h][i] = outlier_val[first + i];
      if (in_tok < TQ_ELL_SLOTS) {
        ell_delta[in_tok * 256 + t] = delta;
        ell_col[in_tok * 256 + t] = (uint8_t)q_row(d);
      } else {
        // (entries are visited in token order, so the list comes out ordered by token)
        for (int q4 = t / 64 + 1; q4 < 5; ++q4) ++ovf_start[q4];
        if (n_ovf < TQ_OVF_CAP) ovf[n_ovf] = ent;
        ++n_ovf;
      }
    }
    for (int q4 = 0; q4 < 5; ++q4) hdr->ovf_start[q4] = (uint16_t)std::min<int>(ovf_start[q4], TQ_OVF_CAP);
    hdr->ovf_n = (uint16_t)std::min(n_ovf, TQ_OVF_CAP);
    // the page's slice of the (layer, seq, head) pool slab, allocated like the encoder does
    uint32_t off = 0;
    int alloc = 0;
    if (n > 0) {
      const int n4 = (n + 3) & ~3;
      off = cursor[h];
      cursor[h] += (uint32_t)n4;
      if (off >= (uint32_t)g.pool_entries) {
        off = 0;
      } else {
        alloc = std::min(n4, g.pool_entries - (int)off);
      }
      if (alloc < n4) pool_short = true;
    }
    meta[h].off = off;
    meta[h].cnt = (uint32_t)std::min(n, alloc);
    hdr->off = meta[h].off;
    hdr->cnt = meta[h].cnt;
    hdr->flags = (n_ovf > TQ_OVF_CAP || alloc < n) ? TQ_PAGE_SPILLED : 0;
  }
  // upload: pages, page metadata, pool entries, cursors
  for (int h = 0; h < H; ++h) {
    TQ_CUDA(cudaMemcpyAsync((uint8_t*)ctx->b.pages + page_offset(g, layer, seq, h, block),
                            pages.data() + (size_t)h * g.page_bytes, g.page_bytes,
                            cudaMemcpyHostToDevice, st));
    const size_t mi = unit_index(g, layer, seq, h) * g.max_blocks + block;
    TQ_CUDA(cudaMemcpyAsync((PageMeta*)ctx->b.page_meta + mi, &meta[h], sizeof(PageMeta),
                            cudaMemcpyHostToDevice, st));
    if (meta[h].cnt > 0) {
      const size_t slab = unit_index(g, layer, seq, h) * (size_t)g.pool_entries + meta[h].off;
      TQ_CUDA(cudaMemcpyAsync((uint32_t*)ctx->b.pool_dec + slab, dec[h].data(), meta[h].cnt * 4,
                              cudaMemcpyHostToDevice, st));
      TQ_CUDA(cudaMemcpyAsync((uint16_t*)ctx->b.pool_val + slab, val[h].data(), meta[h].cnt * 2,
                              cudaMemcpyHostToDevice, st));
    }
  }
  TQ_CUDA(cudaMemcpyAsync(cursor_d, cursor.data(), H * 4, cudaMemcpyHostToDevice, st));
  TQ_CUDA(cudaStreamSynchronize(st));  // the staging vectors go out of scope
  TQ_REQUIRE(!pool_short, TQ_ERR_CAPACITY, "the outlier pool of this sequence is full");
  return TQ_OK;
}

int32_t tq_restore_hot(tq_ctx* ctx, int32_t layer, int32_t seq, int32_t n_tokens,
                       const void* hot_k, const void* hot_v, int64_t tok_stride,
                       int64_t head_stride, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq >= 0 && seq < g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int32_t& len = ctx->len[(size_t)layer * g.n_seqs + seq];
  TQ_REQUIRE(len == 0, TQ_ERR_INVALID, "the cache must be cleared before it is restored");
  TQ_REQUIRE(n_tokens >= 0 && n_tokens <= g.max_tokens_per_seq, TQ_ERR_CAPACITY,
             "n_tokens exceeds max_tokens_per_seq");
  if (n_tokens == 0) return TQ_OK;
  const int nb = n_cold_blocks(n_tokens, g.hot_window, g.block_tokens);
  TQ_REQUIRE(nb <= g.max_blocks, TQ_ERR_CAPACITY, "more cold blocks than the context holds");
  const int hot_start = nb * g.block_tokens, hot_n = n_tokens - hot_start;
  TQ_REQUIRE(hot_k != nullptr && hot_v != nullptr, TQ_ERR_INVALID,
             "hot_k and hot_v must be device pointers");
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  // the ring writer places tokens by position: start it at the first hot position, with no
  // new cold blocks to encode
  int32_t* len_d = (int32_t*)((uint8_t*)ctx->b.state + state_len_off(g)) + layer * g.n_seqs + seq;
  TQ_CUDA(cudaMemcpyAsync(len_d, &hot_start, 4, cudaMemcpyHostToDevice, st));
  TQ_CUDA(cudaStreamSynchronize(st));  // (hot_start is a stack variable)
  int rc = tq_launch_encode(ctx, layer, seq, 1, hot_k, hot_v, hot_n, 0, tok_stride, head_stride,
                            0, st);
  if (rc != TQ_OK) return rc;
  len = n_tokens;
  return TQ_OK;
}

int32_t tq_memory_stats(tq_ctx* ctx, int32_t layer, int32_t seq, double* cold_bytes,
                        double* hot_bytes, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq >= 0 && seq < g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int n = ctx->len[(size_t)layer * g.n_seqs + seq];
  int nb = n_cold_blocks(n, g.hot_window, g.block_tokens);
  const int H = g.n_kv_heads, S = g.block_tokens, D = TQ_D;
  double cold = 0.0;
  if (nb > 0) {
    TQ_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<PageMeta> meta((size_t)H * g.max_blocks);
    TQ_CUDA(cudaMemcpyAsync(
        meta.data(),
        (const PageMeta*)ctx->b.page_meta + unit_index(g, layer, seq, 0) * g.max_blocks,
        meta.size() * sizeof(PageMeta), cudaMemcpyDeviceToHost, st));
    TQ_CUDA(cudaStreamSynchronize(st));
    for (int b = 0; b < nb; ++b) {
      double n_out = 0;
      for (int h = 0; h < H; ++h) n_out += meta[(size_t)h * g.max_blocks + b].cnt;
      if (g.key_mode == TQ_KEYS_POLAR) {
        // a CompressedKV: packed codes + one norm per token
        cold += (double)H * S * D * g.key_bits / 8 + 4.0 * H * S;
      } else {
        // symmetric NF4 containers hold no mean
        cold += (double)H * S * D * g.key_bits / 8 + 4.0 * H * D +
                (g.key_mode == TQ_KEYS_NF4 || ctx->bias_means ? 0.0 : 4.0 * H * ctx->mean_channels) +
                6.0 * n_out;
      }
      cold += (double)H * S * D * g.value_bits / 8 + 4.0 * H * S;
    }
  }
  if (cold_bytes) *cold_bytes = cold;
  if (hot_bytes)
    *hot_bytes = 2.0 * (n - nb * S) * H * D * elem_size(g.kv_dtype);
  return TQ_OK;
}

int32_t tq_clear(tq_ctx* ctx, int32_t layer, int32_t seq, void* stream) {
  TQ_REQUIRE(good_ctx(ctx, layer), TQ_ERR_INVALID, "bad context or layer");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE(seq >= -1 && seq < g.n_seqs, TQ_ERR_INVALID, "bad sequence");
  int s0 = seq < 0 ? 0 : seq, cnt = seq < 0 ? g.n_seqs : 1;
  TQ_CUDA(cudaSetDevice(ctx->device));
  int rc = tq_launch_clear(ctx, layer, s0, cnt, (cudaStream_t)stream);
  if (rc != TQ_OK) return rc;
  for (int s = s0; s < s0 + cnt; ++s) ctx->len[(size_t)layer * g.n_seqs + s] = 0;
  return TQ_OK;
}

int32_t tq_status(tq_ctx* ctx, int32_t* flags, void* stream) {
  TQ_REQUIRE(ctx != nullptr && flags != nullptr, TQ_ERR_INVALID, "null argument");
  TQ_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* d = (int32_t*)((uint8_t*)ctx->b.state + state_status_off(ctx->g));
  TQ_CUDA(cudaMemcpyAsync(flags, d, 4, cudaMemcpyDeviceToHost, st));
  TQ_CUDA(cudaMemsetAsync(d, 0, 4, st));
  TQ_CUDA(cudaStreamSynchronize(st));
  return TQ_OK;
}

int32_t tq_decode_bytes(const tq_ctx* ctx, int32_t layer, double* bytes) {
  TQ_REQUIRE(good_ctx(ctx, layer) && bytes != nullptr, TQ_ERR_INVALID, "bad argument");
  const tq_geom& g = ctx->g;
  const int S = g.block_tokens, D = TQ_D;
  // reference container bytes of one cold block of one KV head, with the nominal
  // outlier count (ties add a few entries that are not counted)
  double blk = (double)S * D * g.key_bits / 8 + (double)S * D * g.value_bits / 8 + 4.0 * S +
               4.0 * D +
               (g.key_mode == TQ_KEYS_NF4 || ctx->bias_means ? 0.0 : 4.0 * ctx->mean_channels) +
               6.0 * g.outlier_k * D;
  double total = 0.0;
  for (int s = 0; s < g.n_seqs; ++s) {
    int n = ctx->len[(size_t)layer * g.n_seqs + s];
    if (n == 0) continue;
    int nb = n_cold_blocks(n, g.hot_window, S);
    total += g.n_kv_heads * (nb * blk + 2.0 * (n - nb * S) * D * elem_size(g.kv_dtype));
    total += (double)g.n_q_heads * D * (elem_size(ctx->last_q_dtype) + 4);
  }
  *bytes = total;
  return TQ_OK;
}

int32_t tq_last_launches(const tq_ctx* ctx) { return ctx ? ctx->last_launches : 0; }

}  // extern "C"
