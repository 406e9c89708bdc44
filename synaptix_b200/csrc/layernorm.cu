// Layer norm (mean and variance, gain and bias) around the residual stream, in 32-bit:
//
//   h_out[t] = h_in[t] + mult * post(delta[t] + dbias)        (post = layer norm with gain pw and bias pb, or the
//                                                              identity when pw is null; nothing is added without delta)
//   y[t]     = ln(h_out[t]) * w + b
//   out[t]   = y[t] + (y'[t] - y[t]) * shift                   (token shift; only with `shift`)
//
// with ln(x) = (x - mean) / sqrt(mean((x - mean)^2) + eps).  y'[t] is the y of the sequence's token before t: the row
// t - 1 of this step, or, for the first row a sequence brings to the step, the row `state[slot]` that the step before
// left (zeros when the slot was opened).  One block computes one row.  With a shift a block forms the y of the row
// before its own a second time instead of waiting for its neighbour, so h_out must not be h_in whenever a sequence
// brings more than one row (the neighbour's h_in is still needed); and the block of a sequence's FIRST row, the only
// one that reads the state, is also the one that writes it (the y of the sequence's last row, formed a third time), so
// no two blocks touch the same state row.
//
// `rows` (without shift): only the listed rows are computed, out is [R, W], and h_out may be null (nothing is
// written back).  delta may be float32 or bfloat16 whatever out is.
#include "common.cuh"

#define LN_THREADS 256

struct LnArgs {
  const float* h_in; float* h_out;
  const void* delta; int delta_dt; const float* dbias;
  const float* pw; const float* pb; float mult;
  const float* w; const float* b; float eps;
  void* out; const int* rows;
  const float* shift; float* state;
  const int* seq_of_token; const int* cu_seqlens; const int* seq_slots;
  int W;
};

// V elements at a time (4 where the width is a multiple of 4: 16-byte loads, so that a row is a few loads a thread and the
// loads of one pass are all in flight together)
template <int V> __device__ __forceinline__ void ln_ld(const float* p, float* f) {
  if (V == 4) { const float4 u = *reinterpret_cast<const float4*>(p); f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w; }
  else f[0] = *p;
}
template <int V> __device__ __forceinline__ void ln_st(float* p, const float* f) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  else *p = f[0];
}
template <int V> __device__ __forceinline__ void ln_st_out(float* p, const float* f) { ln_st<V>(p, f); }
template <int V> __device__ __forceinline__ void ln_st_out(bf16* p, const float* f) {
  if (V == 4) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    *p = __float2bfloat16_rn(f[0]);
  }
}
template <int V> __device__ __forceinline__ void ln_ld_delta(const LnArgs& a, size_t i, float* f) {
  if (a.delta_dt == SX_F32) { ln_ld<V>((const float*)a.delta + i, f); return; }
  const bf16* p = (const bf16*)a.delta + i;
  if (V == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    f[0] = x.x; f[1] = x.y; f[2] = y.x; f[3] = y.y;
  } else {
    f[0] = __bfloat162float(*p);
  }
}

// Block-wide sum with ONE barrier: every warp leaves its sum, and after the barrier every thread adds the warps' sums
// in index order (the same number in every thread).  Two buffers in turn: a thread that writes a buffer again has passed
// the barrier behind the other one, which every thread reaches only after reading this one.
__device__ __forceinline__ float ln_sum(float v, float (*red)[32], int& turn) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  float* r = red[turn];
  turn ^= 1;
  if (lane == 0) r[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nwarp; ++i) s += r[i];
  return s;
}

// the row t after the sum, left in `row` (shared, W floats); returns mean and 1/sqrt(var + eps) of it
template <int V>
__device__ void ln_row(const LnArgs& a, int t, float* row, float (*red)[32], int& turn, float& mean, float& rstd) {
  const int W = a.W, c0 = threadIdx.x * V, step = blockDim.x * V;
  const float invW = 1.f / (float)W;
  const size_t base = (size_t)t * W;
  float s = 0.f;
  if (a.delta) {
    for (int c = c0; c < W; c += step) {
      float d[V], e[V];
      ln_ld_delta<V>(a, base + c, d);
      if (a.dbias) {
        ln_ld<V>(a.dbias + c, e);
#pragma unroll
        for (int i = 0; i < V; ++i) d[i] += e[i];
      }
      ln_st<V>(row + c, d);
#pragma unroll
      for (int i = 0; i < V; ++i) s += d[i];
    }
    if (a.pw) {
      const float mu = ln_sum(s, red, turn) * invW;
      float v = 0.f;
      for (int c = c0; c < W; c += step) {
        float d[V];
        ln_ld<V>(row + c, d);
#pragma unroll
        for (int i = 0; i < V; ++i) v += (d[i] - mu) * (d[i] - mu);
      }
      const float r = rsqrtf(ln_sum(v, red, turn) * invW + a.eps);
      s = 0.f;
      for (int c = c0; c < W; c += step) {
        float d[V], g[V], b[V], h[V];
        ln_ld<V>(row + c, d); ln_ld<V>(a.pw + c, g); ln_ld<V>(a.pb + c, b); ln_ld<V>(a.h_in + base + c, h);
#pragma unroll
        for (int i = 0; i < V; ++i) { d[i] = fmaf(a.mult, fmaf((d[i] - mu) * r, g[i], b[i]), h[i]); s += d[i]; }
        ln_st<V>(row + c, d);
      }
    } else {
      s = 0.f;
      for (int c = c0; c < W; c += step) {
        float d[V], h[V];
        ln_ld<V>(row + c, d); ln_ld<V>(a.h_in + base + c, h);
#pragma unroll
        for (int i = 0; i < V; ++i) { d[i] = fmaf(a.mult, d[i], h[i]); s += d[i]; }
        ln_st<V>(row + c, d);
      }
    }
  } else {
    for (int c = c0; c < W; c += step) {
      float h[V];
      ln_ld<V>(a.h_in + base + c, h);
      ln_st<V>(row + c, h);
#pragma unroll
      for (int i = 0; i < V; ++i) s += h[i];
    }
  }
  mean = ln_sum(s, red, turn) * invW;
  float v = 0.f;
  for (int c = c0; c < W; c += step) {
    float d[V];
    ln_ld<V>(row + c, d);
#pragma unroll
    for (int i = 0; i < V; ++i) v += (d[i] - mean) * (d[i] - mean);
  }
  rstd = rsqrtf(ln_sum(v, red, turn) * invW + a.eps);
}

// the lines of a vector that does not depend on the step before, asked for ahead of the wait for that step
__device__ __forceinline__ void ln_prefetch(const float* p, int W) {
  if (p)
    for (int c = threadIdx.x * 32; c < W; c += blockDim.x * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + c));
}

template <typename TO, int V>
__global__ void __launch_bounds__(1024) add_layernorm_kernel(const LnArgs a) {
  extern __shared__ __align__(16) float ln_smem[];
  __shared__ float red[2][32];
  int turn = 0;
  const int W = a.W;
  ln_prefetch(a.w, W); ln_prefetch(a.b, W); ln_prefetch(a.pw, W); ln_prefetch(a.pb, W); ln_prefetch(a.shift, W);
  ln_prefetch(a.dbias, W);
  pdl_wait();
  pdl_trigger();
  const int c0 = threadIdx.x * V, step = blockDim.x * V;
  float* row = ln_smem;              // this block's row after the sum
  float* other = ln_smem + W;        // a neighbour's (only with a shift)
  const int r = blockIdx.x;
  const int t = a.rows ? a.rows[r] : r;
  float mean, rstd;
  ln_row<V>(a, t, row, red, turn, mean, rstd);
  if (a.h_out && (a.delta || a.h_out != a.h_in))
    for (int c = c0; c < W; c += step) {
      float d[V];
      ln_ld<V>(row + c, d);
      ln_st<V>(a.h_out + (size_t)t * W + c, d);
    }
  TO* out = (TO*)a.out + (size_t)r * W;
  if (!a.shift) {
    for (int c = c0; c < W; c += step) {
      float d[V], g[V], b[V];
      ln_ld<V>(row + c, d); ln_ld<V>(a.w + c, g); ln_ld<V>(a.b + c, b);
#pragma unroll
      for (int i = 0; i < V; ++i) d[i] = fmaf((d[i] - mean) * rstd, g[i], b[i]);
      ln_st_out<V>(out + c, d);
    }
    return;
  }
  const int s = a.seq_of_token[t];
  const int t0 = a.cu_seqlens[s], t1 = a.cu_seqlens[s + 1];
  float* st = a.state + (size_t)a.seq_slots[s] * W;
  if (t > t0) {
    float m2, r2;
    ln_row<V>(a, t - 1, other, red, turn, m2, r2);
    for (int c = c0; c < W; c += step) {
      float d[V], o[V], g[V], b[V], sh[V];
      ln_ld<V>(row + c, d); ln_ld<V>(other + c, o); ln_ld<V>(a.w + c, g); ln_ld<V>(a.b + c, b); ln_ld<V>(a.shift + c, sh);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float y = fmaf((d[i] - mean) * rstd, g[i], b[i]);
        const float yp = fmaf((o[i] - m2) * r2, g[i], b[i]);
        d[i] = fmaf(yp - y, sh[i], y);
      }
      ln_st_out<V>(out + c, d);
    }
    return;
  }
  // the first row a sequence brings: the row before it is the state, and this block leaves the new state
  const bool alone = t1 - t0 == 1;
  float m3 = 0.f, r3 = 0.f;
  if (!alone) ln_row<V>(a, t1 - 1, other, red, turn, m3, r3);
  for (int c = c0; c < W; c += step) {
    float d[V], o[V], g[V], b[V], sh[V], yp[V], ns[V];
    ln_ld<V>(row + c, d); ln_ld<V>(a.w + c, g); ln_ld<V>(a.b + c, b); ln_ld<V>(a.shift + c, sh); ln_ld<V>(st + c, yp);
    if (!alone) ln_ld<V>(other + c, o);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float y = fmaf((d[i] - mean) * rstd, g[i], b[i]);
      d[i] = fmaf(yp[i] - y, sh[i], y);
      ns[i] = alone ? y : fmaf((o[i] - m3) * r3, g[i], b[i]);
    }
    ln_st_out<V>(out + c, d);
    ln_st<V>(st + c, ns);
  }
}

template <typename TO, int V>
static int ln_launch(const LnArgs& a, int R, int threads, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(add_layernorm_kernel<TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return sx_launch(add_layernorm_kernel<TO, V>, dim3(R), dim3(threads), smem, stream, a);
}

extern "C" int sx_add_layernorm(const float* h_in, float* h_out, const void* delta, int delta_dt, const float* dbias,
                                const float* pw, const float* pb, float mult, const float* w, const float* b, float eps,
                                void* out, int out_dt, const int* rows, int R, int W, const float* shift, float* state,
                                const int* seq_of_token, const int* cu_seqlens, const int* seq_slots, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (W <= 0 || W > 24576) return SX_ERR_SIZE;
  if (delta && delta_dt != SX_F32 && delta_dt != SX_BF16) return SX_ERR_DTYPE;
  if (shift && (rows || !state || !seq_of_token || !cu_seqlens || !seq_slots || !h_out)) return SX_ERR_SIZE;
  if ((pw == nullptr) != (pb == nullptr)) return SX_ERR_SIZE;
  LnArgs a;
  a.h_in = h_in; a.h_out = h_out; a.delta = delta; a.delta_dt = delta_dt; a.dbias = dbias; a.pw = pw; a.pb = pb;
  a.mult = mult; a.w = w; a.b = b; a.eps = eps; a.out = out; a.rows = rows; a.shift = shift; a.state = state;
  a.seq_of_token = seq_of_token; a.cu_seqlens = cu_seqlens; a.seq_slots = seq_slots; a.W = W;
  const bool vec = W % 4 == 0 && (((uintptr_t)h_in | (uintptr_t)h_out | (uintptr_t)delta | (uintptr_t)dbias | (uintptr_t)pw |
                               (uintptr_t)pb | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out | (uintptr_t)shift |
                               (uintptr_t)state) & 15) == 0;
  // a thread an element group where the rows are few (a row's loads all in flight at once), else 256 threads a row
  const int groups = vec ? W / 4 : W;
  int threads = R <= 64 ? groups : (groups < LN_THREADS ? groups : LN_THREADS);
  threads = threads > 1024 ? 1024 : (threads + 31) / 32 * 32;
  const size_t smem = (size_t)W * sizeof(float) * (shift ? 2 : 1);
  if (out_dt == SX_F32) return vec ? ln_launch<float, 4>(a, R, threads, smem, stream) : ln_launch<float, 1>(a, R, threads, smem, stream);
  if (out_dt == SX_BF16) return vec ? ln_launch<bf16, 4>(a, R, threads, smem, stream) : ln_launch<bf16, 1>(a, R, threads, smem, stream);
  return SX_ERR_DTYPE;
}
