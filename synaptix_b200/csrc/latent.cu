// Attention over a cached latent (sm_100a), float32 and bfloat16.
//
// A token's cache row is [c | k_rot]: R = kv_rank elements of the normed latent and Dr rotated key elements that all
// heads share; pages are [n_pages, 1, 64, R + Dr].  The keys and values of the heads are never formed: a query is
// taken into the latent's space, attention weights are applied to c itself, and the value matrix of a head is applied
// to the weighted latent.  Queries in the latent's space, scores, softmax and the weighted latents are 32-bit.
//
//   latent_prepare_kernel  one block a token, from the stacked input projection proj [T, row]:
//                          cq = rmsnorm(proj[0:Rq]) * gq  -> cq_out [T, Rq]  (compute dtype)
//                          c  = rmsnorm(proj[col:col+R]) * gkv, k_rot = rotate(proj[col+R : col+R+Dr])  -> the page row
//                          (col < 0 or no pages: the layer reads another layer's cache and writes nothing)
//   latent_query_kernel    one block a (tile of 8 tokens, head): q' = [Wuk_h^T q_h | rotate(q_rot_h)], float32
//                          [T, H, R + Dr]; Wuk is [H * D, R], so q'[r] = sum_d q_h[d] Wuk[h D + d, r]
//   latent_attn_kernel     one block a (token, group of 8 heads), a warp a head: key rows of the window staged in shared
//                          memory 32 at a time for all heads of the block; a lane scores one key, the softmax runs
//                          over the warp, and the weighted sum of c has a lane own the elements r = lane, lane + 32, ...
//                          -> float32 [T, H, splits, R] without the division, and each part's maximum and sum
//   latent_output_kernel   one block a (tile of 8 tokens, head): the parts merged and divided, then
//                          y[h Dv + j] = sigmoid(gate_h) * sum_r Wuv[h Dv + j, r] o'[h, r]
// Rotation: dims elements, pair i at angle position * inv_freq[i]; pairs = 1: elements (2i, 2i + 1), pairs = 0:
// elements (i, i + dims / 2); elements from dims on pass unchanged.  `mag` multiplies cos and sin (1 for a plain rotation;
// a stretched rotation scales both).
#include "common.cuh"
#include <math.h>

#define LT_THREADS 256
#define LT_QTHREADS 128       // threads of a block of the query kernel
#define LT_TOKENS 8          // tokens a block of the query / output kernels
#define LT_HEADS 8           // heads (warps) a block of the attention kernel
#define LT_KEYS 32           // keys staged at a time

__device__ __forceinline__ void rot_pair_index(int i, int dims, int pairs, int& a, int& b) {
  if (pairs) { a = 2 * i; b = 2 * i + 1; } else { a = i; b = i + dims / 2; }
}

template <typename T>
__global__ void __launch_bounds__(LT_THREADS) latent_prepare_kernel(
    const T* __restrict__ proj, int row, int Rq, int col, int R, int Dr, const float* __restrict__ gq,
    const float* __restrict__ gkv, float eps, const float* __restrict__ inv_freq, int dims, int pairs, float mag,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int maxp,
    T* __restrict__ k_pages, T* __restrict__ cq_out) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, tid = threadIdx.x;
  const T* pr = proj + (size_t)t * row;
  float ss = 0.f, inv;
  if (Rq > 0) {                  // a layer whose queries come straight from the projection has no query latent
    for (int i = tid; i < Rq; i += LT_THREADS) { const float v = to_f32(pr[i]); ss += v * v; }
    ss = block_sum(ss, red);
    inv = rsqrtf(ss / (float)Rq + eps);
    for (int i = tid; i < Rq; i += LT_THREADS) cq_out[(size_t)t * Rq + i] = from_f32<T>(to_f32(pr[i]) * inv * gq[i]);
  }
  if (col < 0 || k_pages == nullptr) return;
  const int pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * maxp + (pos >> 6)];
  T* kr = k_pages + ((size_t)page * SX_PAGE + (pos & 63)) * (R + Dr);
  ss = 0.f;
  for (int i = tid; i < R; i += LT_THREADS) { const float v = to_f32(pr[col + i]); ss += v * v; }
  ss = block_sum(ss, red);
  inv = rsqrtf(ss / (float)R + eps);
  for (int i = tid; i < R; i += LT_THREADS) kr[i] = from_f32<T>(to_f32(pr[col + i]) * inv * gkv[i]);
  const T* rr = pr + col + R;
  for (int i = tid; i < dims / 2; i += LT_THREADS) {
    int ia, ib;
    rot_pair_index(i, dims, pairs, ia, ib);
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const float u = to_f32(rr[ia]), v = to_f32(rr[ib]);
    kr[R + ia] = from_f32<T>(u * cs - v * sn);
    kr[R + ib] = from_f32<T>(v * cs + u * sn);
  }
  for (int i = dims + tid; i < Dr; i += LT_THREADS) kr[R + i] = rr[i];
}

extern "C" int sx_latent_prepare(const void* proj, int row, int Rq, int col, int R, int Dr, const float* gq, const float* gkv,
                                 float eps, const float* inv_freq, int dims, int pairs, float mag, const int* positions,
                                 const int* seq_of_token, const int* block_table, int maxp, void* k_pages, void* cq_out,
                                 int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Rq < 0 || (Rq > 0 && (gq == nullptr || cq_out == nullptr)) || dims < 0 || dims > Dr || (dims & 1) || (dims > 0 && inv_freq == nullptr)) return SX_ERR_SIZE;
  if (dt == SX_F32)
    return sx_launch(latent_prepare_kernel<float>, dim3(T), dim3(LT_THREADS), 0, stream, (const float*)proj, row, Rq, col, R, Dr,
                     gq, gkv, eps, inv_freq, dims, pairs, mag, positions, seq_of_token, block_table, maxp, (float*)k_pages, (float*)cq_out);
  if (dt == SX_BF16)
    return sx_launch(latent_prepare_kernel<bf16>, dim3(T), dim3(LT_THREADS), 0, stream, (const bf16*)proj, row, Rq, col, R, Dr,
                     gq, gkv, eps, inv_freq, dims, pairs, mag, positions, seq_of_token, block_table, maxp, (bf16*)k_pages, (bf16*)cq_out);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(LT_QTHREADS) latent_query_kernel(
    const T* __restrict__ q, int QW, const T* __restrict__ wuk, int H, int D, int Dr, int R, const float* __restrict__ inv_freq,
    int dims, int pairs, float mag, const int* __restrict__ positions, float* __restrict__ qa, int n_tokens) {
  extern __shared__ float qs[];          // LT_TOKENS * D; QW: elements between two tokens' queries (>= H (D + Dr))
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.x * LT_TOKENS, h = blockIdx.y, tid = threadIdx.x;
  const int nt = min(LT_TOKENS, n_tokens - t0);
  for (int i = tid; i < LT_TOKENS * D; i += LT_QTHREADS) {
    const int tt = i / D, d = i % D;
    qs[i] = tt < nt ? to_f32(q[(size_t)(t0 + tt) * QW + h * (D + Dr) + d]) : 0.f;
  }
  __syncthreads();
  // the grid's z axis shares the latent's elements: LT_QTHREADS a block
  for (int r = blockIdx.z * LT_QTHREADS + tid; r < min(R, (int)(blockIdx.z + 1) * LT_QTHREADS); r += LT_QTHREADS) {
    float acc[LT_TOKENS];
#pragma unroll
    for (int tt = 0; tt < LT_TOKENS; ++tt) acc[tt] = 0.f;
#pragma unroll 16
    for (int d = 0; d < D; ++d) {
      const float w = to_f32(wuk[((size_t)h * D + d) * R + r]);
#pragma unroll
      for (int tt = 0; tt < LT_TOKENS; ++tt) acc[tt] = fmaf(qs[tt * D + d], w, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < LT_TOKENS; ++tt)
      if (tt < nt) qa[((size_t)(t0 + tt) * H + h) * (R + Dr) + r] = acc[tt];
  }
  if (blockIdx.z != 0) return;
  // the rotated part
  for (int i = tid; i < nt * (dims / 2); i += LT_QTHREADS) {
    const int tt = i / (dims / 2), p = i % (dims / 2);
    int ia, ib;
    rot_pair_index(p, dims, pairs, ia, ib);
    const T* qr = q + (size_t)(t0 + tt) * QW + h * (D + Dr) + D;
    float sn, cs;
    sincosf((float)positions[t0 + tt] * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const float u = to_f32(qr[ia]), v = to_f32(qr[ib]);
    float* o = qa + ((size_t)(t0 + tt) * H + h) * (R + Dr) + R;
    o[ia] = u * cs - v * sn;
    o[ib] = v * cs + u * sn;
  }
  const int rest = Dr - dims;
  for (int i = tid; i < nt * rest; i += LT_QTHREADS) {
    const int tt = i / rest, j = dims + i % rest;
    qa[((size_t)(t0 + tt) * H + h) * (R + Dr) + R + j] = to_f32(q[(size_t)(t0 + tt) * QW + h * (D + Dr) + D + j]);
  }
}

extern "C" int sx_latent_query(const void* q, int q_ld, const void* wuk, int H, int D, int Dr, int R, const float* inv_freq, int dims,
                               int pairs, float mag, const int* positions, float* qa, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_ld < H * (D + Dr)) return SX_ERR_SIZE;
  if (H <= 0 || H > 65535 || D < 0 || R <= 0 || dims < 0 || dims > Dr || (dims & 1)) return SX_ERR_SIZE;
  const size_t smem = (size_t)LT_TOKENS * (D > 0 ? D : 1) * sizeof(float);
  if (smem > 48 * 1024) return SX_ERR_SIZE;
  dim3 grid((T + LT_TOKENS - 1) / LT_TOKENS, H, (R + LT_QTHREADS - 1) / LT_QTHREADS);
  if (dt == SX_F32)
    return sx_launch(latent_query_kernel<float>, grid, dim3(LT_QTHREADS), smem, stream, (const float*)q, q_ld, (const float*)wuk, H, D, Dr,
                     R, inv_freq, dims, pairs, mag, positions, qa, T);
  if (dt == SX_BF16)
    return sx_launch(latent_query_kernel<bf16>, grid, dim3(LT_QTHREADS), smem, stream, (const bf16*)q, q_ld, (const bf16*)wuk, H, D, Dr,
                     R, inv_freq, dims, pairs, mag, positions, qa, T);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
// RI: elements of the weighted latent a lane owns (R <= 32 * RI; with V4, R <= 128 * RI / 4).  The grid's z axis splits the
// window's key tiles among blocks (single-token steps of few sequences would otherwise fill a fraction of the SMs); every
// block writes its weighted sum without the division, out [T, H, splits, R], and its maximum and sum of weights,
// ml [T, H, splits, 2]; the output kernel merges them.
// V4 (R and Dr multiples of 4): staged rows are padded by four floats, so that rows stay 16-byte aligned and the lanes'
// 16-byte loads of different rows fall on different banks; scores take four elements of q and of the key a load, and a
// lane owns the latent's elements 4 lane .. 4 lane + 3 (+ 128, ...), which it reads and writes 16 bytes at a time.
template <typename T, int RI, bool V4>
__global__ void __launch_bounds__(LT_HEADS * 32) latent_attn_kernel(
    const float* __restrict__ qa, const T* __restrict__ k_pages, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int maxp, int H, int R, int Dr, float scale,
    int window, float* __restrict__ out, float* __restrict__ ml) {
  extern __shared__ __align__(16) float sm[];
  const int E = R + Dr, ES = V4 ? E + 4 : E + 1;   // lanes read different rows: the padding spreads them over the banks
  float* ks = sm;                          // LT_KEYS * ES
  float* qs = ks + LT_KEYS * ES;           // LT_HEADS * E
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y * LT_HEADS + warp;
  const int split = blockIdx.z, splits = gridDim.z;
  const bool live = h < H;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)seq_of_token[t] * maxp;
  if (live)
    for (int i = lane; i < E; i += 32) qs[warp * E + i] = qa[((size_t)t * H + h) * E + i];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int tiles = (pos - lo) / LT_KEYS + 1;
  const int per = (tiles + splits - 1) / splits;
  const int j_begin = lo + split * per * LT_KEYS;
  const int j_end = min(pos, lo + (split + 1) * per * LT_KEYS - 1);      // last key of this block
  float m = -INFINITY, l = 0.f;
  float acc[RI];
#pragma unroll
  for (int i = 0; i < RI; ++i) acc[i] = 0.f;
  const float* qh = qs + warp * E;
  for (int j0 = j_begin; j0 <= j_end; j0 += LT_KEYS) {
    const int nk = min(LT_KEYS, j_end - j0 + 1);
    __syncthreads();                        // the tile before is read out (and qs is written)
    constexpr int VEC = 16 / (int)sizeof(T);
    if (E % VEC == 0) {
      // a warp takes whole rows: the page is looked up once a row and the lanes copy 16 bytes each
      for (int jj = warp; jj < nk; jj += LT_HEADS) {
        const int j = j0 + jj;
        const uint4* src = reinterpret_cast<const uint4*>(k_pages + ((size_t)bt[j >> 6] * SX_PAGE + (j & 63)) * E);
        float* dst = ks + jj * ES;
        for (int c = lane; c < E / VEC; c += 32) {
          const uint4 v = src[c];
          const T* x = reinterpret_cast<const T*>(&v);
          if (V4) {
#pragma unroll
            for (int i = 0; i < VEC; i += 4)
              *reinterpret_cast<float4*>(dst + c * VEC + i) = make_float4(to_f32(x[i]), to_f32(x[i + 1]), to_f32(x[i + 2]), to_f32(x[i + 3]));
          } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) dst[c * VEC + i] = to_f32(x[i]);
          }
        }
      }
    } else {
      for (int i = tid; i < nk * E; i += LT_HEADS * 32) {
        const int jj = i / E, e = i % E;
        const int j = j0 + jj;
        ks[jj * ES + e] = to_f32(k_pages[((size_t)bt[j >> 6] * SX_PAGE + (j & 63)) * E + e]);
      }
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * ES;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;      // four sums side by side: the chain of one would wait on itself
      if (V4) {
#pragma unroll 4
        for (int e = 0; e < E; e += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qh + e), k4 = *reinterpret_cast<const float4*>(kr + e);
          d0 = fmaf(q4.x, k4.x, d0); d1 = fmaf(q4.y, k4.y, d1); d2 = fmaf(q4.z, k4.z, d2); d3 = fmaf(q4.w, k4.w, d3);
        }
      } else {
        int e = 0;
        for (; e + 3 < E; e += 4) {
          d0 = fmaf(qh[e], kr[e], d0);
          d1 = fmaf(qh[e + 1], kr[e + 1], d1);
          d2 = fmaf(qh[e + 2], kr[e + 2], d2);
          d3 = fmaf(qh[e + 3], kr[e + 3], d3);
        }
        for (; e < E; ++e) d0 = fmaf(qh[e], kr[e], d0);
      }
      s = ((d0 + d1) + (d2 + d3)) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = lane < nk ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < RI; ++i) acc[i] *= corr;
    for (int jj = 0; jj < nk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* kr = ks + jj * ES;
      if (V4) {
#pragma unroll
        for (int i = 0; i < RI / 4; ++i) {
          const int r = lane * 4 + 128 * i;
          if (r < R) {
            const float4 c4 = *reinterpret_cast<const float4*>(kr + r);
            acc[4 * i] = fmaf(pj, c4.x, acc[4 * i]); acc[4 * i + 1] = fmaf(pj, c4.y, acc[4 * i + 1]);
            acc[4 * i + 2] = fmaf(pj, c4.z, acc[4 * i + 2]); acc[4 * i + 3] = fmaf(pj, c4.w, acc[4 * i + 3]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < RI; ++i) {
          const int r = lane + 32 * i;
          if (r < R) acc[i] = fmaf(pj, kr[r], acc[i]);
        }
      }
    }
  }
  if (live) {
    float* o = out + (((size_t)t * H + h) * splits + split) * R;
    if (V4) {
#pragma unroll
      for (int i = 0; i < RI / 4; ++i) {
        const int r = lane * 4 + 128 * i;
        if (r < R) *reinterpret_cast<float4*>(o + r) = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        const int r = lane + 32 * i;
        if (r < R) o[r] = acc[i];
      }
    }
    if (lane == 0) {
      ml[(((size_t)t * H + h) * splits + split) * 2] = m;
      ml[(((size_t)t * H + h) * splits + split) * 2 + 1] = l;
    }
  }
}

template <typename T, int RI, bool V4>
static int latent_attn_launch(const float* qa, const void* k_pages, const int* positions, const int* seq_of_token,
                              const int* block_table, int maxp, int H, int R, int Dr, float scale, int window, float* out,
                              float* ml, int splits, int T_, cudaStream_t stream) {
  const size_t smem = (size_t)(LT_KEYS * (R + Dr + (V4 ? 4 : 1)) + LT_HEADS * (R + Dr)) * sizeof(float);
  if (smem > 200 * 1024) return SX_ERR_SIZE;
  if (smem > 48 * 1024) cudaFuncSetAttribute(latent_attn_kernel<T, RI, V4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(T_, (H + LT_HEADS - 1) / LT_HEADS, splits);
  return sx_launch(latent_attn_kernel<T, RI, V4>, grid, dim3(LT_HEADS * 32), smem, stream, qa, (const T*)k_pages, positions,
                   seq_of_token, block_table, maxp, H, R, Dr, scale, window, out, ml);
}

template <typename T>
static int latent_attn_any(const float* qa, const void* k_pages, const int* positions, const int* seq_of_token,
                           const int* block_table, int maxp, int H, int R, int Dr, float scale, int window, float* out, float* ml,
                           int splits, int T_, cudaStream_t stream) {
#define LT_CASE(RI, V4) return latent_attn_launch<T, RI, V4>(qa, k_pages, positions, seq_of_token, block_table, maxp, H, R, Dr, scale, window, out, ml, splits, T_, stream)
  if (R % 4 == 0 && Dr % 4 == 0 && (((uintptr_t)qa | (uintptr_t)out) & 15) == 0) {      // a lane owns groups of four elements
    if (R <= 128) LT_CASE(4, true);
    if (R <= 256) LT_CASE(8, true);
    if (R <= 384) LT_CASE(12, true);
    if (R <= 512) LT_CASE(16, true);
    if (R <= 1024) LT_CASE(32, true);
    return SX_ERR_SIZE;
  }
  if (R <= 32 * 2) LT_CASE(2, false);
  if (R <= 32 * 4) LT_CASE(4, false);
  if (R <= 32 * 8) LT_CASE(8, false);
  if (R <= 32 * 12) LT_CASE(12, false);
  if (R <= 32 * 16) LT_CASE(16, false);
  if (R <= 32 * 32) LT_CASE(32, false);
#undef LT_CASE
  return SX_ERR_SIZE;
}

extern "C" int sx_latent_attention(const float* qa, const void* k_pages, const int* positions, const int* seq_of_token,
                                   const int* block_table, int maxp, int H, int R, int Dr, float scale, int window, float* out,
                                   float* ml, int splits, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || R <= 0 || Dr < 0 || (H + LT_HEADS - 1) / LT_HEADS > 65535 || splits < 1 || splits > 64) return SX_ERR_SIZE;
  if (dt == SX_F32) return latent_attn_any<float>(qa, k_pages, positions, seq_of_token, block_table, maxp, H, R, Dr, scale, window, out, ml, splits, T, stream);
  if (dt == SX_BF16) return latent_attn_any<bf16>(qa, k_pages, positions, seq_of_token, block_table, maxp, H, R, Dr, scale, window, out, ml, splits, T, stream);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
#define LT_OUTS 4            // outputs a warp of the output kernel computes side by side

template <typename T>
__global__ void __launch_bounds__(LT_THREADS) latent_output_kernel(
    const float* __restrict__ ol, const float* __restrict__ ml, int splits, const T* __restrict__ wuv, int H, int Dv, int R,
    const T* __restrict__ proj, int row, int col_g, T* __restrict__ y, int n_tokens) {
  extern __shared__ float os[];          // LT_TOKENS * R
  __shared__ float wsp[LT_TOKENS][64];   // each split's weight exp(m_s - M) / L
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.x * LT_TOKENS, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = min(LT_TOKENS, n_tokens - t0);
  if (tid < LT_TOKENS) {
    const int tt = tid;
    if (tt < nt) {
      const float* p = ml + ((size_t)(t0 + tt) * H + h) * splits * 2;
      float M = -INFINITY, L = 0.f;
      for (int s = 0; s < splits; ++s) M = fmaxf(M, p[2 * s]);
      for (int s = 0; s < splits; ++s) L += p[2 * s + 1] * (p[2 * s] == -INFINITY ? 0.f : expf(p[2 * s] - M));
      for (int s = 0; s < splits; ++s) wsp[tt][s] = (p[2 * s] == -INFINITY ? 0.f : expf(p[2 * s] - M)) / L;
    }
  }
  __syncthreads();
#pragma unroll 4                 // the loads of several elements on the way together: they are all the kernel waits for
  for (int i = tid; i < LT_TOKENS * R; i += LT_THREADS) {
    const int tt = i / R, r = i % R;
    float v = 0.f;
    if (tt < nt) {
      const float* p = ol + ((size_t)(t0 + tt) * H + h) * splits * R + r;
#pragma unroll 8
      for (int s = 0; s < splits; ++s) v = fmaf(wsp[tt][s], p[(size_t)s * R], v);
    }
    os[i] = v;
  }
  __syncthreads();
  // the grid's z axis shares the head's outputs: 32 a block
  const int j_hi = min(Dv, (int)(blockIdx.z + 1) * (LT_THREADS / 32) * LT_OUTS);
  for (int j0 = blockIdx.z * (LT_THREADS / 32) * LT_OUTS + warp * LT_OUTS; j0 < j_hi; j0 += (LT_THREADS / 32) * LT_OUTS) {
    float acc[LT_OUTS][LT_TOKENS];
#pragma unroll
    for (int a = 0; a < LT_OUTS; ++a)
#pragma unroll
      for (int tt = 0; tt < LT_TOKENS; ++tt) acc[a][tt] = 0.f;
#pragma unroll 4
    for (int r = lane; r < R; r += 32) {
      float w[LT_OUTS];
#pragma unroll
      for (int a = 0; a < LT_OUTS; ++a) w[a] = j0 + a < Dv ? to_f32(wuv[((size_t)h * Dv + j0 + a) * R + r]) : 0.f;
#pragma unroll
      for (int tt = 0; tt < LT_TOKENS; ++tt) {
        const float x = os[tt * R + r];
#pragma unroll
        for (int a = 0; a < LT_OUTS; ++a) acc[a][tt] = fmaf(x, w[a], acc[a][tt]);
      }
    }
#pragma unroll
    for (int a = 0; a < LT_OUTS; ++a)
#pragma unroll
      for (int tt = 0; tt < LT_TOKENS; ++tt) {
        const float s = warp_sum(acc[a][tt]);
        if (lane == 0 && tt < nt && j0 + a < Dv) {
          float g = 1.f;
          if (col_g >= 0) g = 1.f / (1.f + expf(-to_f32(proj[(size_t)(t0 + tt) * row + col_g + h])));
          y[(size_t)(t0 + tt) * H * Dv + h * Dv + j0 + a] = from_f32<T>(s * g);
        }
      }
  }
}

extern "C" int sx_latent_output(const float* ol, const float* ml, int splits, const void* wuv, int H, int Dv, int R,
                                const void* proj, int row, int col_g, void* y, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || H > 65535 || Dv <= 0 || R <= 0 || splits < 1 || splits > 64) return SX_ERR_SIZE;
  const size_t smem = (size_t)LT_TOKENS * R * sizeof(float);
  if (smem > 48 * 1024) return SX_ERR_SIZE;
  dim3 grid((T + LT_TOKENS - 1) / LT_TOKENS, H, (Dv + (LT_THREADS / 32) * LT_OUTS - 1) / ((LT_THREADS / 32) * LT_OUTS));
  if (dt == SX_F32)
    return sx_launch(latent_output_kernel<float>, grid, dim3(LT_THREADS), smem, stream, ol, ml, splits, (const float*)wuv, H, Dv, R,
                     (const float*)proj, row, col_g, (float*)y, T);
  if (dt == SX_BF16)
    return sx_launch(latent_output_kernel<bf16>, grid, dim3(LT_THREADS), smem, stream, ol, ml, splits, (const bf16*)wuv, H, Dv, R,
                     (const bf16*)proj, row, col_g, (bf16*)y, T);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
// Whole prompts with per-head keys and values (the form that a tensor-core attention kernel over paged keys and values
// takes): the step's latents are gathered from the cache, one product makes every head's unrotated keys and values
// from them, and these kernels lay them out.
//   latent_gather_kernel   c [T, R] and k_rot [T, Dr] of the step's tokens out of their cache rows
//   latent_expand_kernel   kv [T, H * D + H * Dv] (the product's result) and k_rot -> key pages [P, H, 64, D + Dr] =
//                          [k_h | k_rot] and value pages [P, H, 64, Dv], token t of sequence s in page
//                          table[s, pos / 64] at row pos % 64
//   latent_rotate_q_kernel the rotated part of every query head rotated in place ([T, H, D + Dr])
//   head_gate_kernel       y[t, h, :] *= sigmoid(proj[t, col + h])
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ k_pages, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int maxp,
                                     int R, int Dr, T* __restrict__ c, T* __restrict__ kr) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * maxp + (pos >> 6)];
  const T* row = k_pages + ((size_t)page * SX_PAGE + (pos & 63)) * (R + Dr);
  for (int i = threadIdx.x; i < R; i += blockDim.x) c[(size_t)t * R + i] = row[i];
  for (int i = threadIdx.x; i < Dr; i += blockDim.x) kr[(size_t)t * Dr + i] = row[R + i];
}

template <typename T>
__global__ void latent_expand_kernel(const T* __restrict__ kv, const T* __restrict__ kr, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ table, int maxp, int H, int D,
                                     int Dr, int Dv, T* __restrict__ kp, T* __restrict__ vp) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, pos = positions[t];
  const int page = table[(size_t)seq_of_token[t] * maxp + (pos >> 6)];
  const int E = D + Dr, row = pos & 63;
  const T* src = kv + (size_t)t * (H * D + H * Dv);
  constexpr int VEC = 16 / (int)sizeof(T);
  if (D % VEC == 0 && Dr % VEC == 0 && Dv % VEC == 0 && (((uintptr_t)kv | (uintptr_t)kr | (uintptr_t)kp | (uintptr_t)vp) & 15) == 0) {
    const int e4 = E / VEC, d4 = D / VEC, v4 = Dv / VEC;               // 16-byte pieces
    for (int i = threadIdx.x; i < H * e4; i += blockDim.x) {
      const int h = i / e4, e = i % e4;
      const uint4 v = e < d4 ? reinterpret_cast<const uint4*>(src + h * D)[e]
                             : reinterpret_cast<const uint4*>(kr + (size_t)t * Dr)[e - d4];
      reinterpret_cast<uint4*>(kp + (((size_t)page * H + h) * SX_PAGE + row) * E)[e] = v;
    }
    for (int i = threadIdx.x; i < H * v4; i += blockDim.x) {
      const int h = i / v4, e = i % v4;
      reinterpret_cast<uint4*>(vp + (((size_t)page * H + h) * SX_PAGE + row) * Dv)[e] = reinterpret_cast<const uint4*>(src + H * D + h * Dv)[e];
    }
    return;
  }
  for (int i = threadIdx.x; i < H * E; i += blockDim.x) {
    const int h = i / E, e = i % E;
    kp[(((size_t)page * H + h) * SX_PAGE + row) * E + e] = e < D ? src[h * D + e] : kr[(size_t)t * Dr + (e - D)];
  }
  for (int i = threadIdx.x; i < H * Dv; i += blockDim.x) {
    const int h = i / Dv, e = i % Dv;
    vp[(((size_t)page * H + h) * SX_PAGE + row) * Dv + e] = src[H * D + i];
  }
}

template <typename T>
__global__ void latent_rotate_q_kernel(const T* q, int q_ld, T* out, const int* __restrict__ positions,
                                       const float* __restrict__ inv_freq, int dims, int pairs, float mag, int H, int D, int Dr) {
  // out [T, H (D + Dr)] takes the queries with their rotated parts rotated; `q` (rows q_ld apart) may be `out` itself:
  // a thread reads both elements of a pair before it writes them, and copies touch one element each
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dims / 2, HD = D + Dr;
  const T* qi = q + (size_t)t * q_ld;
  T* qo = out + (size_t)t * H * HD;
  if (qi != qo)
    for (int i = threadIdx.x; i < H * HD; i += blockDim.x) {
      const int d = i % HD;
      if (d < D || d >= D + dims) qo[i] = qi[i];
    }
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, p = i % half;
    int ia, ib;
    rot_pair_index(p, dims, pairs, ia, ib);
    const T* qr = qi + h * HD + D;
    float sn, cs;
    sincosf(pos * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const float u = to_f32(qr[ia]), v = to_f32(qr[ib]);
    qo[h * HD + D + ia] = from_f32<T>(u * cs - v * sn);
    qo[h * HD + D + ib] = from_f32<T>(v * cs + u * sn);
  }
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ y, const T* __restrict__ proj, int row, int col, int H, int Dv) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  constexpr int VEC = 16 / (int)sizeof(T);
  if (Dv % VEC == 0 && ((uintptr_t)y & 15) == 0) {
    const int v4 = Dv / VEC;
    for (int i = threadIdx.x; i < H * v4; i += blockDim.x) {
      const float g = 1.f / (1.f + expf(-to_f32(proj[(size_t)t * row + col + i / v4])));
      uint4* p = reinterpret_cast<uint4*>(y + (size_t)t * H * Dv) + i;
      uint4 v = *p;
      T* x = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int k = 0; k < VEC; ++k) x[k] = from_f32<T>(to_f32(x[k]) * g);
      *p = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < H * Dv; i += blockDim.x) {
    const float g = 1.f / (1.f + expf(-to_f32(proj[(size_t)t * row + col + i / Dv])));
    y[(size_t)t * H * Dv + i] = from_f32<T>(to_f32(y[(size_t)t * H * Dv + i]) * g);
  }
}

extern "C" int sx_latent_gather(const void* k_pages, const int* positions, const int* seq_of_token, const int* block_table,
                                int maxp, int R, int Dr, void* c, void* kr, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dt == SX_F32) return sx_launch(latent_gather_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)k_pages, positions, seq_of_token, block_table, maxp, R, Dr, (float*)c, (float*)kr);
  if (dt == SX_BF16) return sx_launch(latent_gather_kernel<bf16>, dim3(T), dim3(256), 0, stream, (const bf16*)k_pages, positions, seq_of_token, block_table, maxp, R, Dr, (bf16*)c, (bf16*)kr);
  return SX_ERR_DTYPE;
}

extern "C" int sx_latent_expand(const void* kv, const void* kr, const int* positions, const int* seq_of_token, const int* table,
                                int maxp, int H, int D, int Dr, int Dv, void* kp, void* vp, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dt == SX_F32) return sx_launch(latent_expand_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)kv, (const float*)kr, positions, seq_of_token, table, maxp, H, D, Dr, Dv, (float*)kp, (float*)vp);
  if (dt == SX_BF16) return sx_launch(latent_expand_kernel<bf16>, dim3(T), dim3(256), 0, stream, (const bf16*)kv, (const bf16*)kr, positions, seq_of_token, table, maxp, H, D, Dr, Dv, (bf16*)kp, (bf16*)vp);
  return SX_ERR_DTYPE;
}

extern "C" int sx_latent_rotate_q(const void* q, int q_ld, void* out, const int* positions, const float* inv_freq, int dims, int pairs,
                                  float mag, int H, int D, int Dr, int T, int dt, cudaStream_t stream) {
  if (T <= 0 || (dims <= 0 && q == out)) return 0;
  if (dims > Dr || (dims & 1) || dims < 0 || q_ld < H * (D + Dr)) return SX_ERR_SIZE;
  if (dt == SX_F32) return sx_launch(latent_rotate_q_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)q, q_ld, (float*)out, positions, inv_freq, dims, pairs, mag, H, D, Dr);
  if (dt == SX_BF16) return sx_launch(latent_rotate_q_kernel<bf16>, dim3(T), dim3(256), 0, stream, (const bf16*)q, q_ld, (bf16*)out, positions, inv_freq, dims, pairs, mag, H, D, Dr);
  return SX_ERR_DTYPE;
}

extern "C" int sx_head_gate(void* y, const void* proj, int row, int col, int H, int Dv, int T, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dt == SX_F32) return sx_launch(head_gate_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)y, (const float*)proj, row, col, H, Dv);
  if (dt == SX_BF16) return sx_launch(head_gate_kernel<bf16>, dim3(T), dim3(256), 0, stream, (bf16*)y, (const bf16*)proj, row, col, H, Dv);
  return SX_ERR_DTYPE;
}
