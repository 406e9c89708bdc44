// Branches that are normed on their way into the residual stream (sm_100a), float32 and bfloat16 branches, all sums
// and norms 32-bit.  One block a row (256 threads, or up to 1,024 where the rows are few); the row stays in shared memory
// between its passes.
//
//   add_normed:   v   = a                                        (one term without a gain; or, with `place`: the weighted
//                       sum of rows of a, sum_k wts[t, k] a[place[t, k]], a mixture of experts' chosen results), or
//                 v   = f * (rms_norm(a) ga + rms_norm(b) gb)     (one or two terms with gains: mixers side by side)
//                 d   = gp ? rms_norm(v) gp : v                   (the branch's own norm)
//                 acc = h ? h[t] + d : d;   if write_h: h[t] = acc
//                 y[r] = go ? rms_norm(acc) go : acc              (the next reader's rows: a cast, or the final norm)
//                 rms_norm(x) = x / sqrt(mean(x^2) + eps).  Rows: r = 0..R-1, t = rows ? rows[r] : r.
//   embed_bigram: out[t] = E[id_t] + B[(prev_t * mp + id_t * mc) mod n], row n of B for a sequence's first token;
//                 prev_t is the token before in the step, or, for a portion's first token, the sequence's state
//                 (its last token), which the same block then moves on to the portion's last token.
#include "common.cuh"

// W elements from a W-aligned place: W = 1, or W = 4 where the width is a multiple of 4 and every array 16-byte aligned
template <int W> __device__ __forceinline__ void ldv(const void* p, int dt, size_t i, float (&v)[W]) {
  if (W == 4) {
    if (dt == SX_F32) {
      const float4 f = *reinterpret_cast<const float4*>((const float*)p + i);
      v[0] = f.x; v[1 % W] = f.y; v[2 % W] = f.z; v[3 % W] = f.w;
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>((const bf16*)p + i);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      v[0] = __low2float(lo); v[1 % W] = __high2float(lo); v[2 % W] = __low2float(hi); v[3 % W] = __high2float(hi);
    }
  } else {
    v[0] = dt == SX_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
  }
}
template <int W> __device__ __forceinline__ void ldfv(const float* p, size_t i, float (&v)[W]) {
  if (W == 4) {
    const float4 f = *reinterpret_cast<const float4*>(p + i);
    v[0] = f.x; v[1 % W] = f.y; v[2 % W] = f.z; v[3 % W] = f.w;
  } else {
    v[0] = p[i];
  }
}
template <int W> __device__ __forceinline__ void stfv(float* p, size_t i, const float (&v)[W]) {
  if (W == 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1 % W], v[2 % W], v[3 % W]);
  else p[i] = v[0];
}
template <int W> __device__ __forceinline__ void stv(float* p, size_t i, const float (&v)[W]) { stfv<W>(p, i, v); }
template <int W> __device__ __forceinline__ void stv(bf16* p, size_t i, const float (&v)[W]) {
  if (W == 4) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1 % W]), hi = __floats2bfloat162_rn(v[2 % W], v[3 % W]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p + i) = u;
  } else {
    p[i] = __float2bfloat16_rn(v[0]);
  }
}

template <typename TO, int W>
__global__ void __launch_bounds__(1024) add_normed_kernel(
    float* __restrict__ h, const void* __restrict__ a, int a_dt, const float* __restrict__ ga,
    const void* __restrict__ b, int b_dt, const float* __restrict__ gb, float factor, const float* __restrict__ gp,
    const float* __restrict__ go, float eps, TO* __restrict__ y, const int* __restrict__ rows, int H, int write_h,
    const int* __restrict__ place, const float* __restrict__ wts, int top) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, tid = threadIdx.x * W, NT = blockDim.x * W;
  const int t = rows ? rows[r] : r;
  const size_t base = (size_t)t * H;
  const float inv_h = 1.f / (float)H;
  float ssv = 0.f;
  float v[W], u[W], g[W];
  if (a == nullptr) {
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] = 0.f;
    for (int i = tid; i < H; i += NT) stfv<W>(row, i, v);
  } else if (ga == nullptr) {
    for (int i = tid; i < H; i += NT) {
      if (place) {                 // the branch is a weighted sum of rows of a (float32), the terms in their order
#pragma unroll
        for (int j = 0; j < W; ++j) v[j] = 0.f;
        for (int k = 0; k < top; ++k) {
          const float wk = wts[(size_t)t * top + k];
          ldfv<W>((const float*)a, (size_t)place[(size_t)t * top + k] * H + i, u);
#pragma unroll
          for (int j = 0; j < W; ++j) v[j] = fmaf(wk, u[j], v[j]);
        }
      } else {
        ldv<W>(a, a_dt, base + i, v);
      }
      stfv<W>(row, i, v);
#pragma unroll
      for (int j = 0; j < W; ++j) ssv += v[j] * v[j];
    }
  } else {
    float sa = 0.f, sb = 0.f;
    for (int i = tid; i < H; i += NT) {
      ldv<W>(a, a_dt, base + i, v);
#pragma unroll
      for (int j = 0; j < W; ++j) sa += v[j] * v[j];
      if (b) {
        ldv<W>(b, b_dt, base + i, u);
#pragma unroll
        for (int j = 0; j < W; ++j) sb += u[j] * u[j];
      }
    }
    sa = block_sum(sa, red);
    const float ra = rsqrtf(sa * inv_h + eps);
    float rb = 0.f;
    if (b) { sb = block_sum(sb, red); rb = rsqrtf(sb * inv_h + eps); }
    for (int i = tid; i < H; i += NT) {
      ldv<W>(a, a_dt, base + i, v);
      ldfv<W>(ga, i, g);
#pragma unroll
      for (int j = 0; j < W; ++j) v[j] = v[j] * ra * g[j];
      if (b) {
        ldv<W>(b, b_dt, base + i, u);
        ldfv<W>(gb, i, g);
#pragma unroll
        for (int j = 0; j < W; ++j) v[j] += u[j] * rb * g[j];
      }
#pragma unroll
      for (int j = 0; j < W; ++j) { v[j] *= factor; ssv += v[j] * v[j]; }
      stfv<W>(row, i, v);
    }
  }
  float rv = 1.f;
  if (gp) { ssv = block_sum(ssv, red); rv = rsqrtf(ssv * inv_h + eps); }
  float ssq = 0.f;
  for (int i = tid; i < H; i += NT) {            // a thread passes over the same elements in every loop: no barrier needed
    ldfv<W>(row, i, v);
    if (gp) {
      ldfv<W>(gp, i, g);
#pragma unroll
      for (int j = 0; j < W; ++j) v[j] = v[j] * rv * g[j];
    }
    if (h) {
      ldfv<W>(h, base + i, u);
#pragma unroll
      for (int j = 0; j < W; ++j) v[j] += u[j];
      if (write_h) stfv<W>(h, base + i, v);
    }
    stfv<W>(row, i, v);
#pragma unroll
    for (int j = 0; j < W; ++j) ssq += v[j] * v[j];
  }
  if (y == nullptr) return;
  TO* yr = y + (size_t)r * H;
  if (go) {
    ssq = block_sum(ssq, red);
    const float ro = rsqrtf(ssq * inv_h + eps);
    for (int i = tid; i < H; i += NT) {
      ldfv<W>(row, i, v);
      ldfv<W>(go, i, g);
#pragma unroll
      for (int j = 0; j < W; ++j) v[j] = v[j] * ro * g[j];
      stv<W>(yr, i, v);
    }
  } else {
    for (int i = tid; i < H; i += NT) {
      ldfv<W>(row, i, v);
      stv<W>(yr, i, v);
    }
  }
}

template <typename TO, int W>
static int add_normed_launch(float* h, const void* a, int a_dt, const float* ga, const void* b, int b_dt, const float* gb,
                             float factor, const float* gp, const float* go, float eps, void* y, const int* rows, int R, int H,
                             int write_h, const int* place, const float* wts, int top, cudaStream_t stream) {
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(add_normed_kernel<TO, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  // few rows (single-token steps): a thread an element or a handful, so that each pass is one trip to memory; many rows:
  // 256 threads a row and several rows an SM
  const int per = (H / W + 31) / 32 * 32;
  const int nt = R <= 296 ? (per > 1024 ? 1024 : (per < 128 ? 128 : per)) : 256;
  return sx_launch(add_normed_kernel<TO, W>, dim3(R), dim3(nt), smem, stream, h, a, a_dt, ga, b, b_dt, gb, factor, gp, go, eps,
                   (TO*)y, rows, H, write_h, place, wts, top);
}

extern "C" int sx_add_normed(float* h, const void* a, int a_dt, const float* ga, const void* b, int b_dt, const float* gb,
                             float factor, const float* gp, const float* go, float eps, void* y, int y_dt, const int* rows,
                             int R, int H, int write_h, const int* place, const float* wts, int top, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || (b != nullptr && (a == nullptr || ga == nullptr || gb == nullptr))) return SX_ERR_SIZE;
  if (place != nullptr && (a == nullptr || a_dt != SX_F32 || ga != nullptr || wts == nullptr || top <= 0)) return SX_ERR_SIZE;
  if ((size_t)H * sizeof(float) > 200 * 1024) return SX_ERR_SIZE;
  const uintptr_t all = (uintptr_t)h | (uintptr_t)a | (uintptr_t)ga | (uintptr_t)b | (uintptr_t)gb | (uintptr_t)gp | (uintptr_t)go |
                        (uintptr_t)y;
  const bool v4 = (H % 4 == 0) && (all % 16 == 0);
#define AN_GO(TO, W) return add_normed_launch<TO, W>(h, a, a_dt, ga, b, b_dt, gb, factor, gp, go, eps, y, rows, R, H, write_h, place, wts, top, stream)
  if (y == nullptr || y_dt == SX_F32) { if (v4) AN_GO(float, 4); AN_GO(float, 1); }
  if (y_dt == SX_BF16) { if (v4) AN_GO(bf16, 4); AN_GO(bf16, 1); }
#undef AN_GO
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
// Only the block of a portion's first token touches its sequence's state: it reads the token before and then stores
// the portion's last token, so no block reads what another writes.  An id outside the table gives zeros for that part.
template <typename T>
__global__ void __launch_bounds__(256) embed_bigram_kernel(
    const T* __restrict__ table, const T* __restrict__ bigram, const int* __restrict__ ids, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
    int* __restrict__ last_token, float* __restrict__ out, int H, int V, int buckets, int mul_prev, int mul_cur) {
  __shared__ int s_prev;
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (threadIdx.x == 0) {
    const int s = seq_of_token[t];
    const int first = cu_seqlens[s];
    int prev;
    if (t == first) {
      const int slot = seq_slots[s];
      prev = last_token[slot];
      last_token[slot] = ids[cu_seqlens[s + 1] - 1];
    } else {
      prev = ids[t - 1];
    }
    s_prev = positions[t] == 0 ? -1 : prev;
  }
  __syncthreads();
  const int prev = s_prev;
  const bool ok = id >= 0 && id < V;
  long long rowb = buckets;                                   // a sequence's first token
  if (prev >= 0) rowb = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
  const T* e = table + (size_t)(ok ? id : 0) * H;
  const T* g = bigram + (size_t)rowb * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_f32(e[i]) + to_f32(g[i]) : 0.f;
}

extern "C" int sx_embed_bigram(const void* table, const void* bigram, int dt, const int* ids, const int* positions,
                               const int* seq_of_token, const int* cu_seqlens, const int* seq_slots, int* last_token, float* out,
                               int n_tokens, int H, int V, int buckets, int mul_prev, int mul_cur, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) return SX_ERR_SIZE;
  if (dt == SX_F32)
    return sx_launch(embed_bigram_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)table, (const float*)bigram, ids,
                     positions, seq_of_token, cu_seqlens, seq_slots, last_token, out, H, V, buckets, mul_prev, mul_cur);
  if (dt == SX_BF16)
    return sx_launch(embed_bigram_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)table, (const bf16*)bigram, ids,
                     positions, seq_of_token, cu_seqlens, seq_slots, last_token, out, H, V, buckets, mul_prev, mul_cur);
  return SX_ERR_DTYPE;
}
