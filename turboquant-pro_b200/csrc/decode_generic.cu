// Decode-on-codes attention, general-shape kernel (any hot_window, any GQA group <= 16,
// float32 arithmetic on the CUDA cores), the split-K combine and the multi-device LSE
// merge.  The tensor-core kernel in decode_mma.cu covers the common geometry and is
// checked against this one.
//
// Score of a cold token, computed on its codes (never materialising K):
//   s = q.mean + sum_d (q_d * scale_d) * NF4[code_d] + sum_{outliers of the token} q_d * delta_d
// Value accumulation stays in the rotated code space, acc_e += p * norm * centroid[code_e];
// the single inverse rotation acc @ Pi is applied once per query head in the combine.
#include "common.cuh"

namespace {

struct DecodeArgs {
  tq_geom g;
  const uint8_t* pages;
  const void* hot_k;
  const void* hot_v;
  const uint32_t* pool_dec;
  const PageMeta* page_meta;
  const int32_t* seq_len;
  const Tables* tables;
  const void* q;
  float* partials;  // [units][max_splits][G][2 + D]
  float* out;       // [n_seqs][n_q_heads][D] or null
  float* mlo;       // [n_seqs][n_q_heads][2 + D] or null
  int layer, q_dtype;
  int ns_cold, ns_hot;
  int block_begin, block_end, with_hot;
  float scale;
};

TQ_DEV float ld_any(const void* p, size_t i, int dt) {
  if (dt == TQ_F32) return ((const float*)p)[i];
  if (dt == TQ_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// 8 consecutive elements starting at element index i (i a multiple of 8)
TQ_DEV void ld8_any(const void* p, size_t i, int dt, float* o) {
  if (dt == TQ_F32) {
    float4 a = *(const float4*)((const float*)p + i);
    float4 b = *(const float4*)((const float*)p + i + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else {
    uint4 r = *(const uint4*)((const uint16_t*)p + i);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (dt == TQ_F16) {
        __half2 h = *(__half2*)&w[k];
        o[2 * k] = __low2float(h);
        o[2 * k + 1] = __high2float(h);
      } else {
        o[2 * k] = __uint_as_float(w[k] << 16);
        o[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
      }
    }
  }
}

constexpr int WARPS = 4;
constexpr int WS = 136;  // padded row stride of the per-page weight table (bank spread)

// One CTA = (split, unit, g-tile).  GT query heads of one KV head are processed together.
template <int GT>
__global__ void __launch_bounds__(WARPS * 32) decode_generic_kernel(DecodeArgs a) {
  const tq_geom& g = a.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, unit = blockIdx.y, gt = blockIdx.z;
  const int seq = unit / g.n_kv_heads, head = unit % g.n_kv_heads;
  const int G = g.group;
  const int S = g.block_tokens, SP = g.block_tokens_pad;
  const int N = a.seq_len[a.layer * g.n_seqs + seq];
  const int nb = n_cold_blocks(N, g.hot_window, S);
  const int hot_start = nb * S, hot_len = N - hot_start;
  const int vb = g.value_bits;

  __shared__ __align__(16) float q_s[GT][TQ_D];
  __shared__ __align__(16) float w_s[GT][WS];
  __shared__ float biasw[WARPS][GT];
  __shared__ float corr_s[GT][256];
  __shared__ float nf4_s[16], cent_s[16];
  __shared__ float p_s[WARPS][GT][TQ_GROUP_TOK];
  __shared__ float ksc_s[WARPS][GT][TQ_GROUP_TOK];  // PolarQuant keys: a group's raw scores
  const bool polar = g.key_mode == TQ_KEYS_POLAR;
  __shared__ float mrg_m[WARPS][GT], mrg_l[WARPS][GT];
  __shared__ float mrg_acc[WARPS][GT][TQ_D];

  if (tid < 16) {
    nf4_s[tid] = a.tables->grid[tid];
    cent_s[tid] = a.tables->centroids[tid];
  }
  for (int i = tid; i < GT * TQ_D; i += WARPS * 32) {
    int gg = i / TQ_D, d = i % TQ_D;
    int qh = gt * GT + gg;
    q_s[gg][d] = qh < G ? ld_any(a.q, ((size_t)seq * g.n_q_heads + head * G + qh) * TQ_D + d,
                                 a.q_dtype)
                        : 0.0f;
  }
  __syncthreads();
  if (polar) {
    // PolarQuant keys (_cold_partials, kv_fused.py:84-98): the score of a token is
    // norm_k * sum_d centroid[code_d] * q_rot[d] with q_rot = q @ Pi^T, formed once here
    // (thread e: column e of Pi^T) and kept where the per-page weights of the per-channel
    // formats go.
    const int e = tid;
    float r[GT];
#pragma unroll
    for (int gg = 0; gg < GT; ++gg) r[gg] = 0.0f;
    for (int d = 0; d < TQ_D; ++d) {
      const float pv = a.tables->pi_t[d * TQ_D + e];
#pragma unroll
      for (int gg = 0; gg < GT; ++gg) r[gg] += q_s[gg][d] * pv;
    }
#pragma unroll
    for (int gg = 0; gg < GT; ++gg) w_s[gg][e] = r[gg];
    __syncthreads();
  }

  float m_run[GT], l_run[GT], acc[GT][16];
#pragma unroll
  for (int gg = 0; gg < GT; ++gg) {
    m_run[gg] = -INFINITY;
    l_run[gg] = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[gg][i] = 0.0f;
  }

  const int tok = lane >> 1, half = lane & 1;  // key-score mapping: 2 lanes per token
  // value mapping: a lane owns 4 tokens and 16 channels (cold codes: dq, dq+8, dq+16, ...;
  // hot rows: 16dq .. 16dq+15)
  const int dq = lane >> 2, c4 = lane & 3;
  const bool cold_split = split < a.ns_cold;

  // online-softmax update of one 16-token group whose raw scores (already scaled, -inf
  // when masked) sit in sc[gg]; leaves p * weight in p_s for the value pass
  auto softmax_step = [&](float* sc, float wgt) {
#pragma unroll
    for (int gg = 0; gg < GT; ++gg) {
      float mx = sc[gg];
#pragma unroll
      for (int o = 16; o >= 2; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float m_new = fmaxf(m_run[gg], mx);
      float p = 0.0f, corr = 1.0f;
      if (m_new > -INFINITY) {
        corr = __expf(m_run[gg] - m_new);
        p = __expf(sc[gg] - m_new);
      }
      l_run[gg] = l_run[gg] * corr + (half == 0 ? p : 0.0f);
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[gg][i] *= corr;
      m_run[gg] = m_new;
      if (half == 0) p_s[warp][gg][tok] = p * wgt;
    }
  };

  // a lane's record of a 16-token group of value-layout codes, and the two codes of its pair p
  auto load_rec = [&](const uint8_t* grp_base, uint32_t (&rec)[8]) {
    if (vb == 4) {
      uint4 r0 = *(const uint4*)(grp_base + lane * 16);
      uint4 r1 = *(const uint4*)(grp_base + 512 + lane * 16);
      rec[0] = r0.x; rec[1] = r0.y; rec[2] = r0.z; rec[3] = r0.w;
      rec[4] = r1.x; rec[5] = r1.y; rec[6] = r1.z; rec[7] = r1.w;
    } else {
#pragma unroll
      for (int pt = 0; pt < 3; ++pt) {
        uint2 r = *(const uint2*)(grp_base + pt * 256 + lane * 8);
        rec[2 * pt] = r.x;
        rec[2 * pt + 1] = r.y;
      }
      rec[6] = rec[7] = 0;
    }
  };
  auto pair_codes = [&](const uint32_t (&rec)[8], int p, int& ca, int& cb) {
    if (vb == 4) {
      uint32_t by = (rec[p >> 2] >> (8 * (p & 3))) & 255;
      ca = by & 15;
      cb = by >> 4;
    } else {
      int bit = 6 * p, wd = bit >> 5, sh = bit & 31;
      uint32_t f = rec[wd] >> sh;
      if (sh > 26) f |= rec[wd + 1] << (32 - sh);
      ca = f & 7;
      cb = (f >> 3) & 7;
    }
  };

  if (split < a.ns_cold) {
    int b0 = min(a.block_begin, nb);
    int b1 = a.block_end < 0 ? nb : min(a.block_end, nb);
    int nbr = max(b1 - b0, 0);
    int p_lo = b0 + (int)((long)nbr * split / a.ns_cold);
    int p_hi = b0 + (int)((long)nbr * (split + 1) / a.ns_cold);
    for (int pg = p_lo; pg < p_hi; ++pg) {
      const uint8_t* page = a.pages + page_offset(g, a.layer, seq, head, pg);
      __syncthreads();
      if (!polar) {  // per-page query projections: w = q * scale, bias = q . mean
        int d = tid;
        float sc = ((const float*)(page + g.scale_off))[d];
        float mu = ((const float*)(page + g.mean_off))[d];
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) {
          float qv = q_s[gg][d];
          w_s[gg][(d >> 6) * 68 + (d & 63)] = qv * sc;
          float b = qv * mu;
#pragma unroll
          for (int o = 16; o >= 1; o >>= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
          if (lane == 0) biasw[warp][gg] = b;
        }
        for (int i = tid; i < GT * 256; i += WARPS * 32) corr_s[i / 256][i % 256] = 0.0f;
      }
      __syncthreads();
      if (!polar) {  // outlier corrections, scattered by token
        PageMeta pm = a.page_meta[unit_index(g, a.layer, seq, head) * g.max_blocks + pg];
        const uint32_t* ent =
            a.pool_dec + unit_index(g, a.layer, seq, head) * (size_t)g.pool_entries + pm.off;
        // The entries are ordered by token, then channel.  The thread that holds a token's first
        // entry adds up all of them in that order, so the sum does not depend on which thread
        // ran first (a float atomic per entry would).
        for (uint32_t e = tid; e < pm.cnt; e += WARPS * 32) {
          const int tk = (int)(ent[e] >> 24);
          if (e > 0 && (int)(ent[e - 1] >> 24) == tk) continue;
          float acc[GT];
#pragma unroll
          for (int gg = 0; gg < GT; ++gg) acc[gg] = 0.0f;
          for (uint32_t j = e; j < pm.cnt; ++j) {
            const uint32_t wv = ent[j];
            if ((int)(wv >> 24) != tk) break;
            const float delta = __half2float(__ushort_as_half((unsigned short)(wv & 0xffff)));
            const int col = (wv >> 16) & 255;
#pragma unroll
            for (int gg = 0; gg < GT; ++gg) acc[gg] += q_s[gg][col] * delta;
          }
#pragma unroll
          for (int gg = 0; gg < GT; ++gg) corr_s[gg][tk] = acc[gg];
        }
      }
      __syncthreads();
      for (int grp = warp; grp < SP / TQ_GROUP_TOK; grp += WARPS) {
        const int t_glob = grp * TQ_GROUP_TOK + tok;
        float sc[GT];
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) sc[gg] = 0.0f;
        if (polar) {
          // key codes in the value layout: this lane's 4 tokens x 16 channels, summed over the
          // eight lanes that share the tokens, then handed to the token's two score lanes
          uint32_t krec[8];
          load_rec(page + (size_t)grp * v_group_bytes(vb), krec);
          float part[4][GT];
#pragma unroll
          for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int gg = 0; gg < GT; ++gg) part[k][gg] = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              int ca, cb;
              pair_codes(krec, 2 * i + h, ca, cb);
              const float va = cent_s[ca], vb2 = cent_s[cb];
#pragma unroll
              for (int gg = 0; gg < GT; ++gg) {
                const float qv = w_s[gg][dq + 8 * i];
                part[2 * h][gg] += va * qv;
                part[2 * h + 1][gg] += vb2 * qv;
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int gg = 0; gg < GT; ++gg) {
              float v = part[k][gg];
              v += __shfl_xor_sync(0xffffffffu, v, 4);
              v += __shfl_xor_sync(0xffffffffu, v, 8);
              v += __shfl_xor_sync(0xffffffffu, v, 16);
              if (dq == 0) ksc_s[warp][gg][2 * c4 + 8 * (k >> 1) + (k & 1)] = v;
            }
          __syncwarp();
        }
        const uint4* row = (const uint4*)(page + (size_t)t_glob * (TQ_D / 2) + half * 32);
#pragma unroll
        for (int v = 0; v < 2 && !polar; ++v) {
          uint4 cw = row[v];
          uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            int dbase = v * 32 + k * 8;  // within this half
            float tv[8];
#pragma unroll
            for (int n = 0; n < 8; ++n) tv[n] = nf4_s[(w4[k] >> (4 * n)) & 15];
#pragma unroll
            for (int gg = 0; gg < GT; ++gg) {
              const float4 wa = *(const float4*)&w_s[gg][half * 68 + dbase];
              const float4 wb = *(const float4*)&w_s[gg][half * 68 + dbase + 4];
              sc[gg] += wa.x * tv[0] + wa.y * tv[1] + wa.z * tv[2] + wa.w * tv[3] +
                        wb.x * tv[4] + wb.y * tv[5] + wb.z * tv[6] + wb.w * tv[7];
            }
          }
        }
        const bool valid = t_glob < S;
        const float nrm = ((const float*)(page + g.norm_off))[t_glob];
        const float nrm_k = polar ? ((const float*)(page + g.scale_off))[t_glob] : 0.0f;
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) {
          float s2 = sc[gg] + __shfl_xor_sync(0xffffffffu, sc[gg], 1);
          if (polar) {
            s2 = nrm_k * ksc_s[warp][gg][tok] * a.scale;
          } else {
            float bias = biasw[0][gg] + biasw[1][gg] + biasw[2][gg] + biasw[3][gg];
            s2 = (s2 + bias + corr_s[gg][t_glob]) * a.scale;
          }
          sc[gg] = valid ? s2 : -INFINITY;
        }
        softmax_step(sc, valid ? nrm : 0.0f);
        __syncwarp();
        // value accumulation on the codes
        const uint8_t* grp_base = page + g.v_off + (size_t)grp * v_group_bytes(vb);
        uint32_t rec[8];
        load_rec(grp_base, rec);
#pragma unroll
        for (int gg = 0; gg < GT; ++gg) {
          float pw[2][2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            pw[h][0] = p_s[warp][gg][2 * c4 + 8 * h];
            pw[h][1] = p_s[warp][gg][2 * c4 + 8 * h + 1];
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              int ca, cb;
              pair_codes(rec, 2 * i + h, ca, cb);
              acc[gg][i] += pw[h][0] * cent_s[ca] + pw[h][1] * cent_s[cb];
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (a.with_hot) {
    const int j = split - a.ns_cold;
    const int ng = (hot_len + TQ_GROUP_TOK - 1) / TQ_GROUP_TOK;
    const int g_lo = (int)((long)ng * j / a.ns_hot), g_hi = (int)((long)ng * (j + 1) / a.ns_hot);
    const int dt = g.kv_dtype;
    const size_t esz = elem_size(dt);
    const uint8_t* hk = (const uint8_t*)a.hot_k + hot_offset_elems(g, a.layer, seq, head) * esz;
    const uint8_t* hv = (const uint8_t*)a.hot_v + hot_offset_elems(g, a.layer, seq, head) * esz;
    for (int grp = g_lo + warp; grp < g_hi; grp += WARPS) {
      const int jt = grp * TQ_GROUP_TOK + tok;
      const bool valid = jt < hot_len;
      float sc[GT];
#pragma unroll
      for (int gg = 0; gg < GT; ++gg) sc[gg] = 0.0f;
      if (valid) {
        const size_t slot = (size_t)((hot_start + jt) % g.hot_cap);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float kv[8];
          ld8_any(hk, slot * TQ_D + half * 64 + k * 8, dt, kv);
#pragma unroll
          for (int gg = 0; gg < GT; ++gg) {
            const float4 qa = *(const float4*)&q_s[gg][half * 64 + k * 8];
            const float4 qb = *(const float4*)&q_s[gg][half * 64 + k * 8 + 4];
            sc[gg] += qa.x * kv[0] + qa.y * kv[1] + qa.z * kv[2] + qa.w * kv[3] +
                      qb.x * kv[4] + qb.y * kv[5] + qb.z * kv[6] + qb.w * kv[7];
          }
        }
      }
#pragma unroll
      for (int gg = 0; gg < GT; ++gg) {
        float s2 = sc[gg] + __shfl_xor_sync(0xffffffffu, sc[gg], 1);
        sc[gg] = valid ? s2 * a.scale : -INFINITY;
      }
      softmax_step(sc, 1.0f);
      __syncwarp();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          const int tl = 2 * c4 + 8 * h + o;
          const int jv = grp * TQ_GROUP_TOK + tl;
          if (jv < hot_len) {
            const size_t slot = (size_t)((hot_start + jv) % g.hot_cap);
            float vv[16];
            ld8_any(hv, slot * TQ_D + dq * 16, dt, vv);
            ld8_any(hv, slot * TQ_D + dq * 16 + 8, dt, vv + 8);
#pragma unroll
            for (int gg = 0; gg < GT; ++gg) {
              const float p = p_s[warp][gg][tl];
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[gg][i] += p * vv[i];
            }
          }
        }
      }
      __syncwarp();
    }
  }

  // lanes that share dq hold different tokens of the same 16 channels
#pragma unroll
  for (int gg = 0; gg < GT; ++gg) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      acc[gg][i] += __shfl_xor_sync(0xffffffffu, acc[gg][i], 1);
      acc[gg][i] += __shfl_xor_sync(0xffffffffu, acc[gg][i], 2);
    }
    float l = l_run[gg];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
      mrg_m[warp][gg] = m_run[gg];
      mrg_l[warp][gg] = l;
    }
    if (c4 == 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        mrg_acc[warp][gg][cold_split ? i * 8 + dq : dq * 16 + i] = acc[gg][i];
    }
  }
  __syncthreads();
  {  // merge the warps' states and store the partial
    const int d = tid;
#pragma unroll
    for (int gg = 0; gg < GT; ++gg) {
      const int qh = gt * GT + gg;
      if (qh >= G) continue;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mrg_m[w][gg]);
      float L = 0.0f, A = 0.0f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float e = mrg_m[w][gg] > -INFINITY ? __expf(mrg_m[w][gg] - M) : 0.0f;
        L += mrg_l[w][gg] * e;
        A += mrg_acc[w][gg][d] * e;
      }
      float* pp = a.partials +
                  (((size_t)unit * g.max_splits + split) * G + qh) * TQ_PART_STRIDE;
      if (d == 0) {
        pp[0] = M;
        pp[1] = L;
      }
      pp[2 + d] = A;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Split-K combine: one CTA per (seq, KV head).  Cold partials are summed in code space and
// un-rotated once (acc @ Pi); hot partials are already in the original basis.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(TQ_D) combine_kernel(DecodeArgs a) {
  const tq_geom& g = a.g;
  const int unit = blockIdx.x, e = threadIdx.x;
  const int seq = unit / g.n_kv_heads, head = unit % g.n_kv_heads;
  const int G = g.group;
  const int ns = a.ns_cold + a.ns_hot;
  __shared__ float cs[TQ_MAX_G][TQ_D];
  __shared__ float sM[TQ_MAX_G], sL[TQ_MAX_G];
  float hot[TQ_MAX_G];
  const float* base = a.partials + (size_t)unit * g.max_splits * G * TQ_PART_STRIDE;
#pragma unroll
  for (int gg = 0; gg < TQ_MAX_G; ++gg) {
    hot[gg] = 0.0f;
    if (gg < G) {
      float M = -INFINITY;
      for (int s = 0; s < ns; ++s) M = fmaxf(M, base[((size_t)s * G + gg) * TQ_PART_STRIDE]);
      float L = 0.0f, C = 0.0f, Hh = 0.0f;
      for (int s = 0; s < ns; ++s) {
        const float* pp = base + ((size_t)s * G + gg) * TQ_PART_STRIDE;
        float w = pp[0] > -INFINITY ? __expf(pp[0] - M) : 0.0f;
        L += pp[1] * w;
        if (s < a.ns_cold)
          C += pp[2 + e] * w;
        else
          Hh += pp[2 + e] * w;
      }
      cs[gg][e] = C;
      hot[gg] = Hh;
      if (e == 0) {
        sM[gg] = M;
        sL[gg] = L;
      }
    }
  }
  __syncthreads();
  float o[TQ_MAX_G];
#pragma unroll
  for (int gg = 0; gg < TQ_MAX_G; ++gg) o[gg] = 0.0f;
  for (int d = 0; d < TQ_D; ++d) {
    const float pv = a.tables->pi[d * TQ_D + e];
#pragma unroll
    for (int gg = 0; gg < TQ_MAX_G; ++gg)
      if (gg < G) o[gg] += cs[gg][d] * pv;
  }
#pragma unroll
  for (int gg = 0; gg < TQ_MAX_G; ++gg) {
    if (gg < G) {
      const size_t row = (size_t)seq * g.n_q_heads + head * G + gg;
      const float val = o[gg] + hot[gg];
      if (a.mlo != nullptr) {
        float* r = a.mlo + row * TQ_PART_STRIDE;
        if (e == 0) {
          r[0] = sM[gg];
          r[1] = sL[gg];
        }
        r[2 + e] = val;
      } else {
        const float L = sL[gg];
        a.out[row * TQ_D + e] = L > 0.0f ? val / L : 0.0f;
      }
    }
  }
}

// Multi-device merge of gathered (m, l, o) states: out = sum_i o_i e^{m_i-M} / sum_i l_i e^{m_i-M},
// parts visited in index order so the result does not depend on arrival order.
__global__ void __launch_bounds__(TQ_D) lse_combine_kernel(const float* mlo, int n_parts,
                                                           int n_rows, float* out) {
  const int row = blockIdx.x, e = threadIdx.x;
  float M = -INFINITY;
  for (int p = 0; p < n_parts; ++p)
    M = fmaxf(M, mlo[((size_t)p * n_rows + row) * TQ_PART_STRIDE]);
  float L = 0.0f, A = 0.0f;
  for (int p = 0; p < n_parts; ++p) {
    const float* r = mlo + ((size_t)p * n_rows + row) * TQ_PART_STRIDE;
    float w = r[0] > -INFINITY ? __expf(r[0] - M) : 0.0f;
    L += r[1] * w;
    A += r[2 + e] * w;
  }
  out[(size_t)row * TQ_D + e] = L > 0.0f ? A / L : 0.0f;
}

template <int GT>
void launch_generic(const DecodeArgs& a, int n_units, cudaStream_t st) {
  dim3 grid(a.ns_cold + a.ns_hot, n_units, (a.g.group + GT - 1) / GT);
  decode_generic_kernel<GT><<<grid, WARPS * 32, 0, st>>>(a);
}

}  // namespace

struct tq_xchg;
int tq_launch_decode_mma(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                         int block_end, int with_hot, float* out, float* mlo, cudaStream_t st,
                         bool* handled, const tq_xchg* xchg, int xchg_phases);

// Sequence-split decode whose merge kernel runs the exchange itself (tensor-core kernel, one
// launch per layer); `handled` tells whether that form was available.
int tq_launch_decode_exchange(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                              int block_end, int with_hot, float* out, const tq_xchg* xchg,
                              int phases, cudaStream_t st, bool* handled) {
  return tq_launch_decode_mma(ctx, layer, q, q_dtype, block_begin, block_end, with_hot, out,
                              nullptr, st, handled, xchg, phases);
}

int tq_launch_decode(tq_ctx* ctx, int layer, const void* q, int q_dtype, int block_begin,
                     int block_end, int with_hot, float* out, float* mlo, cudaStream_t st) {
  const tq_geom& g = ctx->g;
  bool handled = false;
  int rc = tq_launch_decode_mma(ctx, layer, q, q_dtype, block_begin, block_end, with_hot, out,
                                mlo, st, &handled, nullptr, 0);
  if (rc != TQ_OK || handled) return rc;

  DecodeArgs a;
  a.g = g;
  a.pages = (const uint8_t*)ctx->b.pages;
  a.hot_k = ctx->b.hot_k;
  a.hot_v = ctx->b.hot_v;
  a.pool_dec = (const uint32_t*)ctx->b.pool_dec;
  a.page_meta = (const PageMeta*)ctx->b.page_meta;
  a.seq_len = (const int32_t*)((const uint8_t*)ctx->b.state + state_len_off(g));
  a.tables = (const Tables*)ctx->b.tables;
  a.q = q;
  a.partials = (float*)ctx->b.scratch;
  a.out = out;
  a.mlo = mlo;
  a.layer = layer;
  a.q_dtype = q_dtype;
  a.block_begin = block_begin;
  a.block_end = block_end;
  a.with_hot = with_hot;
  a.scale = 1.0f / sqrtf((float)TQ_D);

  // split counts from the longest sequence of the layer: about two pages (or eight hot
  // groups) per CTA, bounded by the scratch slots
  int max_nb = 0, max_hot = 0;
  for (int s = 0; s < g.n_seqs; ++s) {
    int n = ctx->len[(size_t)layer * g.n_seqs + s];
    int nb = n_cold_blocks(n, g.hot_window, g.block_tokens);
    int b1 = block_end < 0 ? nb : std::min(block_end, nb);
    max_nb = std::max(max_nb, std::max(b1 - std::min(block_begin, nb), 0));
    max_hot = std::max(max_hot, n - nb * g.block_tokens);
  }
  int n_units = g.n_seqs * g.n_kv_heads;
  int sm_count = 148;
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, ctx->device);
  int want = std::max(1, (4 * sm_count + n_units - 1) / n_units);  // CTAs per unit to fill the GPU
  int hot_groups = with_hot ? (max_hot + TQ_GROUP_TOK - 1) / TQ_GROUP_TOK : 0;
  int ns_hot = hot_groups > 0 ? std::min(std::min(hot_groups, std::max(1, want / 4)), 16) : 0;
  int ns_cold = max_nb > 0 ? std::min(std::min(max_nb, want), g.max_splits - ns_hot) : 0;
  if (ns_cold + ns_hot == 0) ns_hot = 1;  // empty layer: the kernels still write zeros
  a.ns_cold = ns_cold;
  a.ns_hot = ns_hot;

  cudaEvent_t e0 = tq_prof_event(ctx, 0), e1 = tq_prof_event(ctx, 1), e2 = tq_prof_event(ctx, 2);
  if (e0) cudaEventRecord(e0, st);
  int gt = g.group >= 8 ? 8 : (g.group > 2 ? 4 : (g.group > 1 ? 2 : 1));
  switch (gt) {
    case 1: launch_generic<1>(a, n_units, st); break;
    case 2: launch_generic<2>(a, n_units, st); break;
    case 4: launch_generic<4>(a, n_units, st); break;
    default: launch_generic<8>(a, n_units, st); break;
  }
  if (e1) cudaEventRecord(e1, st);
  combine_kernel<<<n_units, TQ_D, 0, st>>>(a);
  if (e2) {
    cudaEventRecord(e2, st);
    tq_prof_commit(ctx);
  }
  ctx->last_launches = 2;
  ctx->last_kernel = TQ_KERNEL_GENERAL;
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}

int tq_launch_lse_combine(const float* mlo, int n_parts, int n_rows, int head_dim, float* out,
                          cudaStream_t st) {
  (void)head_dim;
  lse_combine_kernel<<<n_rows, TQ_D, 0, st>>>(mlo, n_parts, n_rows, out);
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}

// ---------------------------------------------------------------------------------------
// Decode without caller-provided scratch.
//
// Some embedders cannot give this library any working memory of their own: a plugin that is
// handed only the query and the output tensor by its host engine, a component that runs
// after its process has frozen device allocations for the serving phase, or a sandboxed
// extension that is not allowed to touch the allocator at all.  For them the split-K
// partials live in the fixed array below, which belongs to the library image itself: every
// GPU that loads the library carries these 4.1 MiB until the process exits.
//
// Limits and rules:
//  - at most TQ_STATIC_ROWS (sequence, query head) pairs per call, i.e.
//    n_seqs * n_q_heads <= 1024; larger contexts are refused with TQ_ERR_CAPACITY;
//  - the array is shared by every context and stream of the process on that GPU and keeps
//    whatever the previous call left in it.  Nothing in it has to start at zero: each call
//    overwrites every slot it later reads.  Two calls that run on the GPU at the same time
//    would overwrite each other's partials, so calls must be ordered (same stream, or
//    synchronised);
//  - inside host code the array's name is only a handle; the kernels need its device address.
//    The first call on a device looks that address up (cudaGetSymbolAddress, with that
//    device current) and remembers it, so make the first call on each device before any
//    stream capture begins.
// No allocation happens on this path: no cudaMalloc / cudaFree, no allocating library call.
// ---------------------------------------------------------------------------------------
constexpr int TQ_STATIC_ROWS = 1024;   // most (sequence, query head) pairs per call
constexpr int TQ_STATIC_SLOTS = 8;     // split-K slots per (sequence, KV head)
static __device__ __align__(256) float g_static_partials[(size_t)TQ_STATIC_ROWS * TQ_STATIC_SLOTS *
                                                         TQ_PART_STRIDE];
static float* g_static_partials_addr[64] = {};  // device address of the array, per device

extern "C" int32_t tq_decode_static_scratch(tq_ctx* ctx, int32_t layer, const void* q,
                                            int32_t q_dtype, float* out, void* stream) {
  TQ_REQUIRE(ctx != nullptr && layer >= 0 && layer < ctx->g.n_layers, TQ_ERR_INVALID,
             "bad context or layer");
  TQ_REQUIRE(q != nullptr && out != nullptr, TQ_ERR_INVALID, "q and out must be device pointers");
  TQ_REQUIRE(q_dtype == TQ_F32 || q_dtype == TQ_F16 || q_dtype == TQ_BF16, TQ_ERR_INVALID,
             "bad q_dtype");
  const tq_geom& g = ctx->g;
  TQ_REQUIRE((long)g.n_seqs * g.n_q_heads <= TQ_STATIC_ROWS, TQ_ERR_CAPACITY,
             "tq_decode_static_scratch serves at most 1024 (sequence, query head) pairs "
             "(n_seqs * n_q_heads); use tq_decode with a scratch region for larger contexts");
  TQ_REQUIRE(ctx->device >= 0 && ctx->device < 64, TQ_ERR_INVALID, "device ordinal out of range");
  TQ_CUDA(cudaSetDevice(ctx->device));
  if (g_static_partials_addr[ctx->device] == nullptr) {
    float* p = nullptr;
    TQ_CUDA(cudaGetSymbolAddress((void**)&p, g_static_partials));
    g_static_partials_addr[ctx->device] = p;
  }
  cudaStream_t st = (cudaStream_t)stream;

  DecodeArgs a;
  a.g = g;
  a.g.max_splits = TQ_STATIC_SLOTS;  // slot stride of the partials inside the fixed array
  a.pages = (const uint8_t*)ctx->b.pages;
  a.hot_k = ctx->b.hot_k;
  a.hot_v = ctx->b.hot_v;
  a.pool_dec = (const uint32_t*)ctx->b.pool_dec;
  a.page_meta = (const PageMeta*)ctx->b.page_meta;
  a.seq_len = (const int32_t*)((const uint8_t*)ctx->b.state + state_len_off(g));
  a.tables = (const Tables*)ctx->b.tables;
  a.q = q;
  a.partials = g_static_partials_addr[ctx->device];
  a.out = out;
  a.mlo = nullptr;
  a.layer = layer;
  a.q_dtype = q_dtype;
  a.block_begin = 0;
  a.block_end = -1;
  a.with_hot = 1;
  a.scale = 1.0f / sqrtf((float)TQ_D);

  int max_nb = 0, max_hot = 0;
  for (int s = 0; s < g.n_seqs; ++s) {
    int n = ctx->len[(size_t)layer * g.n_seqs + s];
    int nb = n_cold_blocks(n, g.hot_window, g.block_tokens);
    max_nb = std::max(max_nb, nb);
    max_hot = std::max(max_hot, n - nb * g.block_tokens);
  }
  const int n_units = g.n_seqs * g.n_kv_heads;
  int ns_hot = max_hot > 0 ? std::min((max_hot + 127) / 128, 2) : 0;
  int ns_cold = max_nb > 0 ? std::min(max_nb, TQ_STATIC_SLOTS - ns_hot) : 0;
  if (ns_cold + ns_hot == 0) ns_hot = 1;  // empty layer: the kernels still write zeros
  a.ns_cold = ns_cold;
  a.ns_hot = ns_hot;

  int gt = g.group >= 8 ? 8 : (g.group > 2 ? 4 : (g.group > 1 ? 2 : 1));
  switch (gt) {
    case 1: launch_generic<1>(a, n_units, st); break;
    case 2: launch_generic<2>(a, n_units, st); break;
    case 4: launch_generic<4>(a, n_units, st); break;
    default: launch_generic<8>(a, n_units, st); break;
  }
  combine_kernel<<<n_units, TQ_D, 0, st>>>(a);
  ctx->last_launches = 2;
  ctx->last_kernel = TQ_KERNEL_GENERAL;
  ctx->last_q_dtype = q_dtype;
  TQ_CUDA(cudaGetLastError());
  return TQ_OK;
}
