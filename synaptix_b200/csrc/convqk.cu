// Head preparation of an attention whose queries and keys pass a short causal convolution over time and are normed over
// the whole projection, and whose values are the convolved keys (sm_100a), float32 and bfloat16.
//
//   convqk_prepare  one block a token (256 threads, or up to 1,024 where the tokens are few).  With u the projection's q
//                   and k columns (C = Cq + Ck channels) and taps w [C, n] (handed over taps-major, as [n, C], so that
//                   neighbouring channels' weights of one tap lie together):  y_t[c] = sum_j w[c, j] u_(t - n + 1 + j)[c], the earlier rows taken from the step's own
//                   tokens of the same sequence or, before the portion's start, from the sequence's history (its last
//                   n - 1 projected rows, oldest first; zeros before position 0).
//                   v = y's key channels as they are (the cache's V); q = rms_norm over ALL Cq channels times gq (out),
//                   k = rms_norm over ALL Ck channels times gk (the cache's K).  32-bit sums and norms.
//                   all_single: every sequence brings one token, and the block also moves its history on.
//   convqk_history  otherwise a second launch moves the histories on (blocks of 256 channels a sequence; a thread walks a
//                   channel's rows oldest first, so it reads a row before it overwrites it).
//   sigmoid_gate    y[t, c] *= sigmoid(proj[t, col + c])   (an output gate per element, in place)
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(1024) convqk_prepare_kernel(
    const T* __restrict__ proj, int row, int col_q, int col_k, int Cq, int Ck, int taps, const float* __restrict__ wq,
    const float* __restrict__ wk, const float* __restrict__ gq, const float* __restrict__ gk, float eps, float* __restrict__ hist,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ seq_past,
    const int* __restrict__ seq_slots, const int* __restrict__ block_table, int maxp, T* __restrict__ q_out,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int G, int D, int all_single) {
  extern __shared__ __align__(16) float ys[];       // Cq + Ck convolved values
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, tid = threadIdx.x, NT = blockDim.x;
  const int s = seq_of_token[t], pos = positions[t], past = seq_past[s];
  const int C = Cq + Ck, P = taps - 1;
  float* hs = hist + (size_t)seq_slots[s] * P * C;
  float sq = 0.f, sk = 0.f;
  for (int c = tid; c < C; c += NT) {
    const bool is_q = c < Cq;
    const int pc = is_q ? col_q + c : col_k + (c - Cq);
    const float* w = is_q ? wq + c : wk + (c - Cq);           // taps-major: tap j of this channel lies j * Cx further
    const int wld = is_q ? Cq : Ck;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int p = pos - P + j;                    // the position this tap reads
      if (p < 0) continue;
      float u;
      if (p >= past) u = to_f32(proj[(size_t)(t - (pos - p)) * row + pc]);
      else u = hs[(size_t)(p - past + P) * C + c];
      acc = fmaf(w[(size_t)j * wld], u, acc);
    }
    ys[c] = acc;
    if (is_q) sq += acc * acc; else sk += acc * acc;
    if (all_single && P > 0) {                      // this thread owns the channel's history: shift it by one
      for (int i = 0; i + 1 < P; ++i) hs[(size_t)i * C + c] = hs[(size_t)(i + 1) * C + c];
      hs[(size_t)(P - 1) * C + c] = to_f32(proj[(size_t)t * row + pc]);
    }
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float rq = rsqrtf(sq / (float)Cq + eps), rk = rsqrtf(sk / (float)Ck + eps);
  for (int c = tid; c < Cq; c += NT) q_out[(size_t)t * Cq + c] = from_f32<T>(ys[c] * rq * gq[c]);
  if (k_pages == nullptr) return;
  const int page = block_table[(size_t)s * maxp + (pos >> 6)];
  for (int c = tid; c < Ck; c += NT) {
    const int g = c / D, d = c - g * D;
    const size_t at = (((size_t)page * G + g) * SX_PAGE + (pos & 63)) * D + d;
    const float y = ys[Cq + c];
    k_pages[at] = from_f32<T>(y * rk * gk[c]);
    v_pages[at] = from_f32<T>(y);
  }
}

// eight elements from an 8-aligned place (16 bytes of bfloat16, 32 of float32)
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
}
__device__ __forceinline__ void st8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(bf16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// The same preparation with eight channels a thread at a time: every size and column offset a multiple of 8, every array
// 16-byte aligned, so that all trips to memory are 16 bytes wide.
template <typename T>
__global__ void __launch_bounds__(1024) convqk_prepare_vec_kernel(
    const T* __restrict__ proj, int row, int col_q, int col_k, int Cq, int Ck, int taps, const float* __restrict__ wq,
    const float* __restrict__ wk, const float* __restrict__ gq, const float* __restrict__ gk, float eps, float* __restrict__ hist,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ seq_past,
    const int* __restrict__ seq_slots, const int* __restrict__ block_table, int maxp, T* __restrict__ q_out,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int G, int D, int all_single) {
  extern __shared__ __align__(16) float ys[];       // Cq + Ck convolved values
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, tid = threadIdx.x, NT = blockDim.x;
  const int s = seq_of_token[t], pos = positions[t], past = seq_past[s];
  const int C = Cq + Ck, P = taps - 1;
  float* hs = hist + (size_t)seq_slots[s] * P * C;
  float sq = 0.f, sk = 0.f;
  for (int c0 = tid * 8; c0 < C; c0 += NT * 8) {
    const bool is_q = c0 < Cq;
    const int pc = is_q ? col_q + c0 : col_k + (c0 - Cq);
    const float* w = is_q ? wq + c0 : wk + (c0 - Cq);         // taps-major: eight channels' weights of a tap lie together
    const int wld = is_q ? Cq : Ck;
    float acc[8], u[8], wj[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int p = pos - P + j;                    // the position this tap reads
      if (p < 0) continue;
      if (p >= past) ld8(proj + (size_t)(t - (pos - p)) * row + pc, u);
      else ld8(hs + (size_t)(p - past + P) * C + c0, u);
      ld8(w + (size_t)j * wld, wj);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(wj[e], u[e], acc[e]);
    }
    st8(ys + c0, acc);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += acc[e] * acc[e];
    if (is_q) sq += ss; else sk += ss;
    if (all_single && P > 0) {                      // this thread owns these channels' history: shift it by one
      for (int i = 0; i + 1 < P; ++i) {
        ld8(hs + (size_t)(i + 1) * C + c0, u);
        st8(hs + (size_t)i * C + c0, u);
      }
      ld8(proj + (size_t)t * row + pc, u);
      st8(hs + (size_t)(P - 1) * C + c0, u);
    }
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float rq = rsqrtf(sq / (float)Cq + eps), rk = rsqrtf(sk / (float)Ck + eps);
  float y[8], g[8];
  for (int c0 = tid * 8; c0 < Cq; c0 += NT * 8) {
    ld8(ys + c0, y);
    ld8(gq + c0, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = y[e] * rq * g[e];
    st8(q_out + (size_t)t * Cq + c0, y);
  }
  if (k_pages == nullptr) return;
  const int page = block_table[(size_t)s * maxp + (pos >> 6)];
  for (int c0 = tid * 8; c0 < Ck; c0 += NT * 8) {
    const int gi = c0 / D, d = c0 - gi * D;          // D is a multiple of 8: the eight channels lie in one head
    const size_t at = (((size_t)page * G + gi) * SX_PAGE + (pos & 63)) * D + d;
    ld8(ys + Cq + c0, y);
    st8(v_pages + at, y);
    ld8(gk + c0, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = y[e] * rk * g[e];
    st8(k_pages + at, y);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) convqk_history_kernel(const T* __restrict__ proj, int row, int col_q, int col_k, int Cq, int Ck,
                                                             int taps, float* __restrict__ hist, const int* __restrict__ cu_seqlens,
                                                             const int* __restrict__ seq_slots) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x;
  const int t0 = cu_seqlens[s], n = cu_seqlens[s + 1] - t0;
  const int C = Cq + Ck, P = taps - 1;
  if (n <= 0) return;
  float* hs = hist + (size_t)seq_slots[s] * P * C;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < C; c += gridDim.y * 256) {
    const int pc = c < Cq ? col_q + c : col_k + (c - Cq);
    for (int i = 0; i < P; ++i) {                   // new row i is row i + n of [old rows ++ the step's rows]
      const int src = i + n;
      hs[(size_t)i * C + c] = src < P ? hs[(size_t)src * C + c] : to_f32(proj[(size_t)(t0 + src - P) * row + pc]);
    }
  }
}

extern "C" int sx_convqk_prepare(const void* proj, int row, int col_q, int col_k, int Cq, int Ck, int taps, const float* wq,
                                 const float* wk, const float* gq, const float* gk, float eps, float* hist, const int* positions,
                                 const int* seq_of_token, const int* cu_seqlens, const int* seq_past, const int* seq_slots,
                                 const int* block_table, int maxp, void* q_out, void* k_pages, void* v_pages, int G, int D,
                                 int n_tokens, int n_seqs, int all_single, int dt, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || Cq <= 0 || Ck <= 0 || G * D != Ck || col_q < 0 || col_k < 0 || col_q + Cq > row || col_k + Ck > row)
    return SX_ERR_SIZE;
  const size_t smem = (size_t)(Cq + Ck) * sizeof(float);
  if (smem > 48 * 1024) return SX_ERR_SIZE;
  // few tokens (single-token steps): a thread walks a handful of channels, each a chain of dependent trips to memory
  const int C = Cq + Ck;
  const int nt = n_tokens <= 296 ? (C >= 2048 ? 1024 : (C >= 1024 ? 512 : 256)) : 256;
  const int hist_blocks = (C + 255) / 256 < 64 ? (C + 255) / 256 : 64;
  const uintptr_t all = (uintptr_t)proj | (uintptr_t)wq | (uintptr_t)wk | (uintptr_t)gq | (uintptr_t)gk | (uintptr_t)hist |
                        (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages;
  const bool vec = ((row | col_q | col_k | Cq | Ck | D) % 8 == 0) && all % 16 == 0;
  const int ntv = n_tokens <= 296 ? (C >= 4096 ? 512 : 256) : 128;         // eight channels a thread
  int rc;
  if (vec && dt == SX_F32)
    rc = sx_launch(convqk_prepare_vec_kernel<float>, dim3(n_tokens), dim3(ntv), smem, stream, (const float*)proj, row, col_q, col_k,
                   Cq, Ck, taps, wq, wk, gq, gk, eps, hist, positions, seq_of_token, seq_past, seq_slots, block_table, maxp,
                   (float*)q_out, (float*)k_pages, (float*)v_pages, G, D, all_single);
  else if (vec && dt == SX_BF16)
    rc = sx_launch(convqk_prepare_vec_kernel<bf16>, dim3(n_tokens), dim3(ntv), smem, stream, (const bf16*)proj, row, col_q, col_k,
                   Cq, Ck, taps, wq, wk, gq, gk, eps, hist, positions, seq_of_token, seq_past, seq_slots, block_table, maxp,
                   (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, G, D, all_single);
  else if (dt == SX_F32)
    rc = sx_launch(convqk_prepare_kernel<float>, dim3(n_tokens), dim3(nt), smem, stream, (const float*)proj, row, col_q, col_k, Cq,
                   Ck, taps, wq, wk, gq, gk, eps, hist, positions, seq_of_token, seq_past, seq_slots, block_table, maxp,
                   (float*)q_out, (float*)k_pages, (float*)v_pages, G, D, all_single);
  else if (dt == SX_BF16)
    rc = sx_launch(convqk_prepare_kernel<bf16>, dim3(n_tokens), dim3(nt), smem, stream, (const bf16*)proj, row, col_q, col_k, Cq,
                   Ck, taps, wq, wk, gq, gk, eps, hist, positions, seq_of_token, seq_past, seq_slots, block_table, maxp,
                   (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages, G, D, all_single);
  else
    return SX_ERR_DTYPE;
  if (rc || all_single || taps == 1) return rc;
  if (dt == SX_F32)
    return sx_launch(convqk_history_kernel<float>, dim3(n_seqs, hist_blocks), dim3(256), 0, stream, (const float*)proj, row, col_q, col_k, Cq, Ck,
                     taps, hist, cu_seqlens, seq_slots);
  return sx_launch(convqk_history_kernel<bf16>, dim3(n_seqs, hist_blocks), dim3(256), 0, stream, (const bf16*)proj, row, col_q, col_k, Cq, Ck,
                   taps, hist, cu_seqlens, seq_slots);
}

// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ y, const T* __restrict__ proj, int row, int col, int n, size_t total) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / n;
  const int c = (int)(idx - t * n);
  const float g = to_f32(proj[t * row + col + c]);
  y[idx] = from_f32<T>(to_f32(y[idx]) / (1.f + expf(-g)));
}
// eight elements a thread (n, row and col multiples of 8, both arrays 16-byte aligned); total counts groups of eight
template <typename T>
__global__ void sigmoid_gate_vec_kernel(T* __restrict__ y, const T* __restrict__ proj, int row, int col, int n, size_t total) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per = n / 8;
  const size_t t = idx / per;
  const int c = (int)(idx - t * per) * 8;
  float v[8], g[8];
  ld8(y + t * n + c, v);
  ld8(proj + t * row + col + c, g);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = v[e] / (1.f + expf(-g[e]));
  st8(y + t * n + c, v);
}

extern "C" int sx_sigmoid_gate(void* y, const void* proj, int row, int col, int n, int n_tokens, int dt, cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * n;
  if (total == 0) return 0;
  if (col < 0 || col + n > row) return SX_ERR_SIZE;
  if (((row | col | n) % 8 == 0) && ((uintptr_t)y | (uintptr_t)proj) % 16 == 0) {
    const size_t groups = total / 8;
    const dim3 grid((unsigned)((groups + 255) / 256));
    if (dt == SX_F32) return sx_launch(sigmoid_gate_vec_kernel<float>, grid, dim3(256), 0, stream, (float*)y, (const float*)proj, row, col, n, groups);
    if (dt == SX_BF16) return sx_launch(sigmoid_gate_vec_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)y, (const bf16*)proj, row, col, n, groups);
    return SX_ERR_DTYPE;
  }
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dt == SX_F32) return sx_launch(sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, (float*)y, (const float*)proj, row, col, n, total);
  if (dt == SX_BF16) return sx_launch(sigmoid_gate_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)y, (const bf16*)proj, row, col, n, total);
  return SX_ERR_DTYPE;
}
