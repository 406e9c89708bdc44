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

__device__ __forceinline__ float ln_load_delta(const LnArgs& a, size_t i) {
  return a.delta_dt == SX_F32 ? ((const float*)a.delta)[i] : __bfloat162float(((const bf16*)a.delta)[i]);
}

// the row t after the sum, left in `row` (shared, W floats); returns mean and 1/sqrt(var + eps) of it
__device__ void ln_row(const LnArgs& a, int t, float* row, float* red, float& mean, float& rstd) {
  const int W = a.W;
  const float invW = 1.f / (float)W;
  const size_t base = (size_t)t * W;
  if (a.delta) {
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float d = ln_load_delta(a, base + c) + (a.dbias ? a.dbias[c] : 0.f);
      row[c] = d;
      s += d;
    }
    if (a.pw) {
      const float mu = block_sum(s, red) * invW;
      float v = 0.f;
      for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = row[c] - mu; v += d * d; }
      const float r = rsqrtf(block_sum(v, red) * invW + a.eps);
      for (int c = threadIdx.x; c < W; c += blockDim.x)
        row[c] = fmaf(a.mult, fmaf((row[c] - mu) * r, a.pw[c], a.pb[c]), a.h_in[base + c]);
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) row[c] = fmaf(a.mult, row[c], a.h_in[base + c]);
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) row[c] = a.h_in[base + c];
  }
  float s = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) s += row[c];
  mean = block_sum(s, red) * invW;
  float v = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = row[c] - mean; v += d * d; }
  rstd = rsqrtf(block_sum(v, red) * invW + a.eps);
}

template <typename TO>
__global__ void __launch_bounds__(LN_THREADS) add_layernorm_kernel(const LnArgs a) {
  extern __shared__ float ln_smem[];
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int W = a.W;
  float* row = ln_smem;              // this block's row after the sum
  float* other = ln_smem + W;        // a neighbour's (only with a shift)
  const int r = blockIdx.x;
  const int t = a.rows ? a.rows[r] : r;
  float mean, rstd;
  ln_row(a, t, row, red, mean, rstd);
  if (a.h_out && a.delta)
    for (int c = threadIdx.x; c < W; c += blockDim.x) a.h_out[(size_t)t * W + c] = row[c];
  else if (a.h_out && a.h_out != a.h_in)
    for (int c = threadIdx.x; c < W; c += blockDim.x) a.h_out[(size_t)t * W + c] = row[c];
  TO* out = (TO*)a.out + (size_t)r * W;
  if (!a.shift) {
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[c] = from_f32<TO>(fmaf((row[c] - mean) * rstd, a.w[c], a.b[c]));
    return;
  }
  const int s = a.seq_of_token[t];
  const int t0 = a.cu_seqlens[s], t1 = a.cu_seqlens[s + 1];
  float* st = a.state + (size_t)a.seq_slots[s] * W;
  if (t > t0) {
    float m2, r2;
    ln_row(a, t - 1, other, red, m2, r2);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float y = fmaf((row[c] - mean) * rstd, a.w[c], a.b[c]);
      const float yp = fmaf((other[c] - m2) * r2, a.w[c], a.b[c]);
      out[c] = from_f32<TO>(fmaf(yp - y, a.shift[c], y));
    }
    return;
  }
  // the first row a sequence brings: the row before it is the state, and this block leaves the new state
  const bool alone = t1 - t0 == 1;
  float m3 = 0.f, r3 = 0.f;
  if (!alone) ln_row(a, t1 - 1, other, red, m3, r3);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float y = fmaf((row[c] - mean) * rstd, a.w[c], a.b[c]);
    const float yp = st[c];
    out[c] = from_f32<TO>(fmaf(yp - y, a.shift[c], y));
    st[c] = alone ? y : fmaf((other[c] - m3) * r3, a.w[c], a.b[c]);
  }
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
  const int threads = W <= 128 ? 64 : (W <= 1024 ? 128 : LN_THREADS);
  const size_t smem = (size_t)W * sizeof(float) * (shift ? 2 : 1);
  if (out_dt == SX_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(add_layernorm_kernel<float>, dim3(R), dim3(threads), smem, stream, a);
  }
  if (out_dt == SX_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sx_launch(add_layernorm_kernel<bf16>, dim3(R), dim3(threads), smem, stream, a);
  }
  return SX_ERR_DTYPE;
}
