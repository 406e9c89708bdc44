// Kernels of parts that carry something from token to token besides keys and values: a short causal convolution
// over time in front of a sublayer, a gated recurrence per channel (minGRU), linear attention with a fixed decay per
// head (retention), and the small elementwise steps around them (a capped gated activation, vectors added into the
// residual stream).  Float32 and bfloat16 storage; positions, norms, gates, decays, states and every sum are 32-bit.
//
// Tokens of all sequences of a step are packed into one stream, as everywhere in this package: token t belongs to
// row s = seq_of_token[t] of the per-sequence arrays, the tokens of s are cu_seqlens[s] .. cu_seqlens[s+1]-1 and stand
// at positions seq_past[s] .. seq_lens[s]-1.  A state lives in a tensor [slots, ...] in 32-bit, indexed by
// seq_slots[s]; a slot is zeroed when a sequence opens it.  Nothing here needs a value of the step on the host, so
// every kernel can be recorded into a CUDA graph.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f32(float x) { return x / (1.f + expf(-x)); }

// ---------------------------------------------------------------------------------------
// Residual sum + RMSNorm in front of a short convolution.
//   rows 0..T-1:        v = h[t] (+ delta[t], written back);  y[t] = v * rsqrt(mean(v^2) + eps) * w     (32-bit out)
//   rows T..T+S*P-1:    y[T + s*P + i] = hist[slot(s)][i]   (P = taps - 1: the last P inputs of the sequence before
//                       this step, oldest first), so that the convolution reads one buffer and may write hist.
// ---------------------------------------------------------------------------------------
template <typename TD>
__global__ void __launch_bounds__(256) add_rmsnorm_hist_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                               const float* __restrict__ w, float eps, float* __restrict__ y,
                                                               const float* __restrict__ hist, const int* __restrict__ seq_slots,
                                                               int T, int P, int H) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x;
  if (b >= T) {
    const int s = (b - T) / P, i = (b - T) % P;
    const float* src = hist + ((size_t)seq_slots[s] * P + i) * H;
    float* dst = y + (size_t)b * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
    return;
  }
  float* hr = h + (size_t)b * H;
  const TD* dr = delta ? delta + (size_t)b * H : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = hr[c];
    if (dr) {
      v += to_f32(dr[c]);
      hr[c] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  float* yr = y + (size_t)b * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) yr[c] = hr[c] * inv * w[c];
}

extern "C" int sx_add_rmsnorm_hist(float* h, const void* delta, int delta_dt, const float* w, float eps, float* y,
                                   const float* hist, const int* seq_slots, int T, int S, int P, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (P < 0 || H <= 0) return SX_ERR_SIZE;
  const dim3 grid(T + S * P);
  if (delta_dt == SX_F32)
    return sx_launch(add_rmsnorm_hist_kernel<float>, grid, dim3(256), 0, stream, h, (const float*)delta, w, eps, y, hist,
                     seq_slots, T, P, H);
  if (delta_dt == SX_BF16)
    return sx_launch(add_rmsnorm_hist_kernel<bf16>, grid, dim3(256), 0, stream, h, (const bf16*)delta, w, eps, y, hist,
                     seq_slots, T, P, H);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// Short causal convolution over time on each channel, added to its input:
//   out[t] = y[t] + sum_{j < taps} cw[c][j] * y_at(position(t) - (taps-1) + j)
// y is the buffer of the kernel above: an input at a position of this step is a row of the step, an older one a
// history row (zeros before the sequence's start, since a fresh slot's history is zero).  The block of a sequence's
// last token of the step writes the new history (the last P inputs, oldest first).
// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256) token_conv_kernel(const float* __restrict__ y, const float* __restrict__ cw,
                                                         TO* __restrict__ out, float* __restrict__ hist,
                                                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_past,
                                                         const int* __restrict__ seq_lens, const int* __restrict__ seq_slots,
                                                         int T, int P, int H) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int s = seq_of_token[t], pos = positions[t];
  const int start = seq_past[s], t0 = cu_seqlens[s], end = seq_lens[s];
  const int taps = P + 1;
  // row of y that holds the input at position p (start - P <= p <= pos)
  auto row_of = [&](int p) -> size_t { return p >= start ? (size_t)(t0 + (p - start)) : (size_t)(T + s * P + (p - start + P)); };
  if ((H & 3) == 0) {                                        // four channels a thread, 16 bytes a load
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(y + (size_t)t * H + c);
      for (int j = 0; j < taps; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(y + row_of(pos - P + j) * H + c);
        a.x = fmaf(cw[(size_t)c * taps + j], v.x, a.x);
        a.y = fmaf(cw[(size_t)(c + 1) * taps + j], v.y, a.y);
        a.z = fmaf(cw[(size_t)(c + 2) * taps + j], v.z, a.z);
        a.w = fmaf(cw[(size_t)(c + 3) * taps + j], v.w, a.w);
      }
      TO* o = out + (size_t)t * H + c;
      o[0] = from_f32<TO>(a.x); o[1] = from_f32<TO>(a.y); o[2] = from_f32<TO>(a.z); o[3] = from_f32<TO>(a.w);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float acc = y[(size_t)t * H + c];
      for (int j = 0; j < taps; ++j) acc = fmaf(cw[(size_t)c * taps + j], y[row_of(pos - P + j) * H + c], acc);
      out[(size_t)t * H + c] = from_f32<TO>(acc);
    }
  }
  if (pos == end - 1) {
    float* hs = hist + (size_t)seq_slots[s] * P * H;
    for (int i = 0; i < P; ++i) {
      const size_t r = row_of(end - P + i);
      for (int c = threadIdx.x; c < H; c += blockDim.x) hs[(size_t)i * H + c] = y[r * H + c];
    }
  }
}

extern "C" int sx_token_conv(const float* y, const float* cw, void* out, int out_dt, float* hist, const int* positions,
                             const int* seq_of_token, const int* cu_seqlens, const int* seq_past, const int* seq_lens,
                             const int* seq_slots, int T, int P, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (P < 0 || H <= 0) return SX_ERR_SIZE;
  if (out_dt == SX_F32)
    return sx_launch(token_conv_kernel<float>, dim3(T), dim3(256), 0, stream, y, cw, (float*)out, hist, positions, seq_of_token,
                     cu_seqlens, seq_past, seq_lens, seq_slots, T, P, H);
  if (out_dt == SX_BF16)
    return sx_launch(token_conv_kernel<bf16>, dim3(T), dim3(256), 0, stream, y, cw, (bf16*)out, hist, positions, seq_of_token,
                     cu_seqlens, seq_past, seq_lens, seq_slots, T, P, H);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// The two kernels above as one, for steps in which every sequence brings ONE token (row t is sequence t):
// sum, norm, convolution over the history and the history's shift, one block a token.  Rows of up to
// 256 * NC channels stay in registers.
// ---------------------------------------------------------------------------------------
template <typename TD, int NC>
__global__ void __launch_bounds__(1024) norm_conv_step_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                              const float* __restrict__ w, float eps, const float* __restrict__ cw,
                                                              TD* __restrict__ out, float* __restrict__ hist,
                                                              const int* __restrict__ seq_slots, int P, int H) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, nt = blockDim.x;
  float* __restrict__ hr = h + (size_t)t * H;
  const TD* __restrict__ dr = delta ? delta + (size_t)t * H : nullptr;
  float v[NC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NC; ++k) {
    const int c = threadIdx.x + k * nt;
    v[k] = 0.f;
    if (c < H) {
      v[k] = hr[c];
      if (dr) {
        v[k] += to_f32(dr[c]);
        hr[c] = v[k];
      }
      ss += v[k] * v[k];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  const int taps = P + 1;
  float* __restrict__ hs = hist + (size_t)seq_slots[t] * P * H;
#pragma unroll
  for (int k = 0; k < NC; ++k) {
    const int c = threadIdx.x + k * nt;
    if (c >= H) continue;
    const float yv = v[k] * inv * w[c];
    const float* __restrict__ cwc = cw + (size_t)c * taps;
    float acc = fmaf(cwc[P], yv, yv);
    float prev = yv;                        // walks the history from the newest entry down, shifting it by one
    for (int i = P - 1; i >= 0; --i) {
      const float old = hs[(size_t)i * H + c];
      acc = fmaf(cwc[i], old, acc);
      hs[(size_t)i * H + c] = prev;
      prev = old;
    }
    out[(size_t)t * H + c] = from_f32<TD>(acc);
  }
}

extern "C" int sx_norm_conv_step(float* h, const void* delta, const float* w, float eps, const float* cw, void* out,
                                 float* hist, const int* seq_slots, int T, int P, int H, int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (P < 0 || H <= 0 || H > 1024 * 8) return SX_ERR_SIZE;
  // a token's row is one block's: as many threads as the row has channels, up to 1,024, then several channels a thread
  const int threads = H >= 1024 ? 1024 : ((H + 31) / 32) * 32;
#define NCS_GO(TD, NC)                                                                                                  \
  return sx_launch(norm_conv_step_kernel<TD, NC>, dim3(T), dim3(threads), 0, stream, h, (const TD*)delta, w, eps, cw, (TD*)out, \
                   hist, seq_slots, P, H)
#define NCS_PICK(TD)              \
  if (H <= threads) NCS_GO(TD, 1);     \
  if (H <= threads * 2) NCS_GO(TD, 2); \
  if (H <= threads * 4) NCS_GO(TD, 4); \
  NCS_GO(TD, 8)
  if (dt == SX_F32) { NCS_PICK(float); }
  if (dt == SX_BF16) { NCS_PICK(bf16); }
#undef NCS_PICK
#undef NCS_GO
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// minGRU: per channel c of N,  z = sigmoid(a_z + b_z),  u = a_x + b_x,  cand = u >= 0 ? u + 1/2 : sigmoid(u),
//   S <- (1 - z) S + z cand,   out = S * silu(a_g),
// where a_z, a_x, a_g are columns z_off + c, x_off + c, g_off + c of the projection `proj` [T, row].
//
// mingru_scan_kernel walks a sequence's tokens one after the other, a thread a channel: single-token steps and
// short portions.  Longer portions go through three kernels that cut a sequence's tokens into pieces of CH:
//   (1) a piece composed from a zero state: (A, B) with S_end = A S_begin + B, per piece and channel;
//   (2) the pieces' carries one after the other (few), which also leaves the sequence's new state;
//   (3) every piece again from its true begin state, writing the outputs.
// ---------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void mingru_gate(const T* __restrict__ row, int z_off, int x_off, int c, float bz, float bx,
                                            float& keep, float& add) {
  const float z = sigmoid_f32(to_f32(row[z_off + c]) + bz);
  const float u = to_f32(row[x_off + c]) + bx;
  const float cand = u >= 0.f ? u + 0.5f : sigmoid_f32(u);
  keep = 1.f - z;
  add = z * cand;
}

template <typename T>
__global__ void __launch_bounds__(128) mingru_scan_kernel(const T* __restrict__ proj, int row, int z_off, int x_off, int g_off,
                                                          const float* __restrict__ bz, const float* __restrict__ bx,
                                                          float* __restrict__ state, T* __restrict__ out,
                                                          const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
                                                          int N) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= N) return;
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  float* sp = state + (size_t)seq_slots[s] * N + c;
  float S = *sp;
  const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const T* r = proj + (size_t)t * row;
    float keep, add;
    mingru_gate(r, z_off, x_off, c, b_z, b_x, keep, add);
    S = fmaf(keep, S, add);
    out[(size_t)t * N + c] = from_f32<T>(S * silu_f32(to_f32(r[g_off + c])));
  }
  *sp = S;
}

#define MG_CH 64
// every SEQUENCE is cut into pieces of its own (piece k of sequence s covers its tokens 64 k .. 64 k + 63 of this step),
// so no piece crosses a border between sequences; the grid is (most pieces of a sequence, sequences, channel blocks) and
// pieces beyond a sequence's end return at once.  AB: [S, max_pieces, 2, N].
template <typename T>
__global__ void __launch_bounds__(128) mingru_piece_kernel(const T* __restrict__ proj, int row, int z_off, int x_off,
                                                           const float* __restrict__ bz, const float* __restrict__ bx,
                                                           float* __restrict__ AB, const int* __restrict__ cu_seqlens,
                                                           int N, int max_pieces) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.y, p = blockIdx.x, c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = cu_seqlens[s] + p * MG_CH, t1 = min(cu_seqlens[s + 1], t0 + MG_CH);
  if (c >= N || t0 >= t1) return;
  const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
  float A = 1.f, B = 0.f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    float keep, add;
    mingru_gate(proj + (size_t)t * row, z_off, x_off, c, b_z, b_x, keep, add);
    A *= keep;
    B = fmaf(keep, B, add);
  }
  float* ab = AB + (((size_t)s * max_pieces + p) * 2) * N;
  ab[c] = A;
  ab[N + c] = B;
}

// the begin state of every piece (written over A) and the sequence's new state
__global__ void __launch_bounds__(128) mingru_carry_kernel(float* __restrict__ AB, float* __restrict__ state,
                                                           const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots,
                                                           int N, int max_pieces) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= N) return;
  const int n = cu_seqlens[s + 1] - cu_seqlens[s];
  const int pieces = (n + MG_CH - 1) / MG_CH;
  float* sp = state + (size_t)seq_slots[s] * N + c;
  float S = *sp;
  for (int p0 = 0; p0 < pieces; p0 += 8) {                 // eight pieces' (A, B) on the way at once, then the chain
    float A[8], B[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float* ab = AB + (((size_t)s * max_pieces + min(p0 + k, pieces - 1)) * 2) * N;
      A[k] = ab[c];
      B[k] = ab[N + c];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (p0 + k < pieces) {
        AB[(((size_t)s * max_pieces + p0 + k) * 2) * N + c] = S;
        S = fmaf(A[k], S, B[k]);
      }
  }
  *sp = S;
}

template <typename T>
__global__ void __launch_bounds__(128) mingru_apply_kernel(const T* __restrict__ proj, int row, int z_off, int x_off, int g_off,
                                                           const float* __restrict__ bz, const float* __restrict__ bx,
                                                           const float* __restrict__ AB, T* __restrict__ out,
                                                           const int* __restrict__ cu_seqlens, int N, int max_pieces) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.y, p = blockIdx.x, c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = cu_seqlens[s] + p * MG_CH, t1 = min(cu_seqlens[s + 1], t0 + MG_CH);
  if (c >= N || t0 >= t1) return;
  const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
  float S = AB[(((size_t)s * max_pieces + p) * 2) * N + c];
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const T* r = proj + (size_t)t * row;
    float keep, add;
    mingru_gate(r, z_off, x_off, c, b_z, b_x, keep, add);
    S = fmaf(keep, S, add);
    out[(size_t)t * N + c] = from_f32<T>(S * silu_f32(to_f32(r[g_off + c])));
  }
}

// The piece and apply kernels for projections whose rows and columns allow 16-byte loads: a block brings the 64 x 128
// tile of each of its columns' arrays into shared memory with every thread's loads on the way at once, and a thread
// then walks its channel there (a thread that fetches its own channel token by token has a few bytes in flight).
#define MG_TC 128
template <typename T, bool APPLY>
__global__ void __launch_bounds__(MG_TC) mingru_tile_kernel(const T* __restrict__ proj, int row, int z_off, int x_off, int g_off,
                                                            const float* __restrict__ bz, const float* __restrict__ bx,
                                                            float* __restrict__ AB, T* __restrict__ out,
                                                            const int* __restrict__ cu_seqlens, int N, int max_pieces) {
  extern __shared__ __align__(16) unsigned char mg_smem[];
  T* zs = reinterpret_cast<T*>(mg_smem);
  T* xs = zs + MG_CH * MG_TC;
  T* gs = xs + MG_CH * MG_TC;
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.y, p = blockIdx.x, c0 = blockIdx.z * MG_TC, tid = threadIdx.x, c = c0 + tid;
  const int t0 = cu_seqlens[s] + p * MG_CH, n = min(cu_seqlens[s + 1] - t0, MG_CH);
  if (n <= 0) return;
  constexpr int V = 16 / (int)sizeof(T), VPR = MG_TC / V;          // elements a load, loads a tile row
  const int ncol = min(MG_TC, N - c0);                              // N is a multiple of V: a load is whole or absent
  for (int idx = tid; idx < n * VPR; idx += MG_TC) {
    const int j = idx / VPR, col = (idx % VPR) * V;
    if (col >= ncol) continue;
    const T* src = proj + (size_t)(t0 + j) * row + c0 + col;
    *reinterpret_cast<uint4*>(zs + j * MG_TC + col) = *reinterpret_cast<const uint4*>(src + z_off);
    *reinterpret_cast<uint4*>(xs + j * MG_TC + col) = *reinterpret_cast<const uint4*>(src + x_off);
    if (APPLY) *reinterpret_cast<uint4*>(gs + j * MG_TC + col) = *reinterpret_cast<const uint4*>(src + g_off);
  }
  __syncthreads();
  if (c >= N) return;
  const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
  float* ab = AB + (((size_t)s * max_pieces + p) * 2) * N;
  if (!APPLY) {
    float A = 1.f, B = 0.f;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
      const float z = sigmoid_f32(to_f32(zs[j * MG_TC + tid]) + b_z);
      const float u = to_f32(xs[j * MG_TC + tid]) + b_x;
      const float keep = 1.f - z, add = z * (u >= 0.f ? u + 0.5f : sigmoid_f32(u));
      A *= keep;
      B = fmaf(keep, B, add);
    }
    ab[c] = A;
    ab[N + c] = B;
  } else {
    float S = ab[c];
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
      const float z = sigmoid_f32(to_f32(zs[j * MG_TC + tid]) + b_z);
      const float u = to_f32(xs[j * MG_TC + tid]) + b_x;
      S = fmaf(1.f - z, S, z * (u >= 0.f ? u + 0.5f : sigmoid_f32(u)));
      out[(size_t)(t0 + j) * N + c] = from_f32<T>(S * silu_f32(to_f32(gs[j * MG_TC + tid])));
    }
  }
}

template <typename T>
static int mingru_launch(const void* proj, int row, int z_off, int x_off, int g_off, const float* bz, const float* bx,
                         float* state, void* out, float* scratch, const int* cu_seqlens, const int* seq_slots, int S, int N,
                         int max_new, cudaStream_t stream) {
  const int cb = (N + 127) / 128;
  if (max_new <= 2 * MG_CH || scratch == nullptr)
    return sx_launch(mingru_scan_kernel<T>, dim3(S, cb), dim3(128), 0, stream, (const T*)proj, row, z_off, x_off, g_off, bz, bx,
                     state, (T*)out, cu_seqlens, seq_slots, N);
  const int max_pieces = (max_new + MG_CH - 1) / MG_CH;
  constexpr int V = 16 / (int)sizeof(T);
  if (row % V == 0 && z_off % V == 0 && x_off % V == 0 && g_off % V == 0 && N % V == 0 && ((uintptr_t)proj & 15) == 0) {
    const dim3 grid(max_pieces, S, (N + MG_TC - 1) / MG_TC);
    const size_t tile = (size_t)MG_CH * MG_TC * sizeof(T);
    if (3 * tile > 48 * 1024) {
      cudaError_t ce = cudaFuncSetAttribute(mingru_tile_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(3 * tile));
      if (ce != cudaSuccess) return (int)ce;
      ce = cudaFuncSetAttribute(mingru_tile_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * tile));
      if (ce != cudaSuccess) return (int)ce;
    }
    int e = sx_launch(mingru_tile_kernel<T, false>, grid, dim3(MG_TC), 2 * tile, stream, (const T*)proj, row, z_off, x_off, g_off, bz,
                      bx, scratch, (T*)out, cu_seqlens, N, max_pieces);
    if (e) return e;
    e = sx_launch(mingru_carry_kernel, dim3(S, cb), dim3(128), 0, stream, scratch, state, cu_seqlens, seq_slots, N, max_pieces);
    if (e) return e;
    return sx_launch(mingru_tile_kernel<T, true>, grid, dim3(MG_TC), 3 * tile, stream, (const T*)proj, row, z_off, x_off, g_off, bz, bx,
                     scratch, (T*)out, cu_seqlens, N, max_pieces);
  }
  int e = sx_launch(mingru_piece_kernel<T>, dim3(max_pieces, S, cb), dim3(128), 0, stream, (const T*)proj, row, z_off, x_off, bz,
                    bx, scratch, cu_seqlens, N, max_pieces);
  if (e) return e;
  e = sx_launch(mingru_carry_kernel, dim3(S, cb), dim3(128), 0, stream, scratch, state, cu_seqlens, seq_slots, N, max_pieces);
  if (e) return e;
  return sx_launch(mingru_apply_kernel<T>, dim3(max_pieces, S, cb), dim3(128), 0, stream, (const T*)proj, row, z_off, x_off, g_off,
                   bz, bx, (const float*)scratch, (T*)out, cu_seqlens, N, max_pieces);
}

// scratch: float32 [S, ceil(max_new / 64), 2, N], or null (then the sequential kernel runs whatever the length)
extern "C" int sx_mingru(const void* proj, int row, int z_off, int x_off, int g_off, const float* bz, const float* bx,
                         float* state, void* out, float* scratch, const int* cu_seqlens, const int* seq_slots, int S, int N,
                         int max_new, int dt, cudaStream_t stream) {
  if (S <= 0 || N <= 0) return 0;
  if (S > 65535) return SX_ERR_SIZE;
  if (dt == SX_F32)
    return mingru_launch<float>(proj, row, z_off, x_off, g_off, bz, bx, state, out, scratch, cu_seqlens, seq_slots, S, N, max_new, stream);
  if (dt == SX_BF16)
    return mingru_launch<bf16>(proj, row, z_off, x_off, g_off, bz, bx, state, out, scratch, cu_seqlens, seq_slots, S, N, max_new, stream);
  return SX_ERR_DTYPE;
}
extern "C" int sx_mingru_piece_tokens() { return MG_CH; }

// ---------------------------------------------------------------------------------------
// Retention: linear attention with a fixed decay per head, no softmax and no denominator.  Per head, with
// q, k of size D and v of size E (columns q_off + head*D, k_off + head*D, v_off + head*E of `proj` [T, row]):
//   S <- decay S + (k * kscale) v^T   ([D, E], 32-bit, state [slots, heads, D, E]),   o = S^T q,
//   out[t, head*E + e] = o[e] / sqrt(mean_e(o^2) + eps) * silu(gate[t, g_off + head*E + e]) * out_scale
// (the gate and the unit norm are optional).  One block per (sequence, head) walks the sequence's tokens; S lies in
// shared memory; thread (g, e) owns column e and the rows d = g, g + G, ... of S.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024) retention_kernel(const T* __restrict__ proj, int row, int q_off, int k_off, int v_off,
                                                        int g_off, const float* __restrict__ decay, float kscale, float eps,
                                                        int unit_norm, float out_scale, float* __restrict__ state,
                                                        T* __restrict__ out, int out_stride, const int* __restrict__ cu_seqlens,
                                                        const int* __restrict__ seq_slots, int heads, int D, int E) {
  extern __shared__ float sm[];
  float* S = sm;                     // D * E
  float* qs = S + (size_t)D * E;     // D
  float* ks = qs + D;                // D
  float* vs = ks + D;                // E
  float* part = vs + E;              // G * E
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x, hd = blockIdx.y, tid = threadIdx.x;
  const int G = blockDim.x / E;                      // E <= blockDim.x is checked by the host
  const int e = tid % E, g = tid / E;
  const bool live = g < G;
  const float dc = decay[hd];
  float* sp = state + ((size_t)seq_slots[s] * heads + hd) * D * E;
  for (int i = tid; i < D * E; i += blockDim.x) S[i] = sp[i];
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  for (int t = t0; t < t1; ++t) {
    const T* r = proj + (size_t)t * row;
    __syncthreads();                                  // the token before is done with qs, ks, vs, part
    for (int i = tid; i < D; i += blockDim.x) {
      qs[i] = to_f32(r[q_off + hd * D + i]);
      ks[i] = to_f32(r[k_off + hd * D + i]) * kscale;
    }
    for (int i = tid; i < E; i += blockDim.x) vs[i] = to_f32(r[v_off + hd * E + i]);
    __syncthreads();
    if (live) {
      const float ve = vs[e];
      float acc = 0.f;
      for (int d = g; d < D; d += G) {
        const float x = fmaf(dc, S[d * E + e], ks[d] * ve);
        S[d * E + e] = x;
        acc = fmaf(x, qs[d], acc);
      }
      part[g * E + e] = acc;
    }
    __syncthreads();
    float o = 0.f;
    if (tid < E)
      for (int i = 0; i < G; ++i) o += part[i * E + tid];
    float inv = 1.f;
    if (unit_norm) inv = rsqrtf(block_sum(tid < E ? o * o : 0.f, red) / (float)E + eps);
    if (tid < E) {
      float x = o * inv;
      if (g_off >= 0) x *= silu_f32(to_f32(r[g_off + hd * E + tid]));
      out[(size_t)t * out_stride + hd * E + tid] = from_f32<T>(x * out_scale);
    }
  }
  __syncthreads();
  for (int i = tid; i < D * E; i += blockDim.x) sp[i] = S[i];
}

extern "C" int sx_retention(const void* proj, int row, int q_off, int k_off, int v_off, int g_off, const float* decay,
                            float kscale, float eps, int unit_norm, float out_scale, float* state, void* out, int out_stride,
                            const int* cu_seqlens, const int* seq_slots, int S, int heads, int D, int E, int dt,
                            cudaStream_t stream) {
  if (S <= 0 || heads <= 0) return 0;
  if (D <= 0 || E <= 0 || E > 1024 || heads > 65535) return SX_ERR_SIZE;
  const int threads = E <= 256 ? 256 : (E <= 512 ? 512 : 1024);        // a thread a value element at least
  const int G = threads / E;
  const size_t smem = ((size_t)D * E + 2 * D + E + (size_t)G * E) * sizeof(float);
  if (smem > 200 * 1024) return SX_ERR_SIZE;
  const dim3 grid(S, heads);
#define RET_GO(TT)                                                                                                          \
  {                                                                                                                         \
    if (smem > 48 * 1024) {                                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(retention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                                  \
    }                                                                                                                       \
    return sx_launch(retention_kernel<TT>, grid, dim3(threads), smem, stream, (const TT*)proj, row, q_off, k_off, v_off, g_off, \
                     decay, kscale, eps, unit_norm, out_scale, state, (TT*)out, out_stride, cu_seqlens, seq_slots, heads, D, E); \
  }
  if (dt == SX_F32) RET_GO(float)
  if (dt == SX_BF16) RET_GO(bf16)
#undef RET_GO
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// Retention for steps of ONE token a sequence (row t is sequence t): the state is read from and written back to
// global memory directly, every element once, without a stop in shared memory.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024) retention_step_kernel(const T* __restrict__ proj, int row, int q_off, int k_off, int v_off,
                                                             int g_off, const float* __restrict__ decay, float kscale, float eps,
                                                             int unit_norm, float out_scale, float* __restrict__ state,
                                                             T* __restrict__ out, int out_stride, const int* __restrict__ seq_slots,
                                                             int heads, int D, int E) {
  extern __shared__ float sm[];
  float* qs = sm;            // D
  float* ks = qs + D;        // D
  float* part = ks + D;      // G * E
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, hd = blockIdx.y, tid = threadIdx.x;
  const int G = blockDim.x / E, e = tid % E, g = tid / E;
  const T* r = proj + (size_t)t * row;
  for (int i = tid; i < D; i += blockDim.x) {
    qs[i] = to_f32(r[q_off + hd * D + i]);
    ks[i] = to_f32(r[k_off + hd * D + i]) * kscale;
  }
  __syncthreads();
  if (g < G) {
    const float dc = decay[hd], ve = to_f32(r[v_off + hd * E + e]);
    float* sp = state + ((size_t)seq_slots[t] * heads + hd) * D * E + e;
    float acc = 0.f;
    int d = g;
    for (; d + 3 * G < D; d += 4 * G) {                 // four rows at a time: their loads are on the way together
      float x0 = sp[(size_t)d * E], x1 = sp[(size_t)(d + G) * E], x2 = sp[(size_t)(d + 2 * G) * E], x3 = sp[(size_t)(d + 3 * G) * E];
      x0 = fmaf(dc, x0, ks[d] * ve); x1 = fmaf(dc, x1, ks[d + G] * ve);
      x2 = fmaf(dc, x2, ks[d + 2 * G] * ve); x3 = fmaf(dc, x3, ks[d + 3 * G] * ve);
      sp[(size_t)d * E] = x0; sp[(size_t)(d + G) * E] = x1; sp[(size_t)(d + 2 * G) * E] = x2; sp[(size_t)(d + 3 * G) * E] = x3;
      acc = fmaf(x0, qs[d], acc); acc = fmaf(x1, qs[d + G], acc); acc = fmaf(x2, qs[d + 2 * G], acc); acc = fmaf(x3, qs[d + 3 * G], acc);
    }
    for (; d < D; d += G) {
      const float x = fmaf(dc, sp[(size_t)d * E], ks[d] * ve);
      sp[(size_t)d * E] = x;
      acc = fmaf(x, qs[d], acc);
    }
    part[g * E + e] = acc;
  }
  __syncthreads();
  float o = 0.f;
  if (tid < E)
    for (int i = 0; i < G; ++i) o += part[i * E + tid];
  float inv = 1.f;
  if (unit_norm) inv = rsqrtf(block_sum(tid < E ? o * o : 0.f, red) / (float)E + eps);
  if (tid < E) {
    float x = o * inv;
    if (g_off >= 0) x *= silu_f32(to_f32(r[g_off + hd * E + tid]));
    out[(size_t)t * out_stride + hd * E + tid] = from_f32<T>(x * out_scale);
  }
}

// ---------------------------------------------------------------------------------------
// Retention over long portions, in pieces of RC tokens a sequence (counted from the portion's first token), three kernels:
//   (1) a piece's own sum U = sum_j decay^(n-1-j) k_j v_j^T (n tokens in the piece), per (piece, head, sequence);
//   (2) the pieces' begin states one after the other: S_(c+1) = decay^n S_c + U_c, written over U; the last is the new state;
//   (3) a piece's outputs: o_i = sum_{j<=i} decay^(i-j) (q_i . k_j) v_j + decay^(i+1) S_c^T q_i, then unit norm, gate, store.
// All products are 32-bit FFMA on tiles in shared memory: 256 threads as 16 x 16, 4 x 4 results a thread, operands as
// At[k][m] and B[k][n] with leading sizes that are multiples of 4 (padding zeroed), so both are read 16 bytes at a time.
// ---------------------------------------------------------------------------------------
#define RC 64
__host__ __device__ static inline int up4(int x) { return (x + 3) & ~3; }

template <typename F>
__device__ __forceinline__ void tile_product2(const float* __restrict__ At1, int lda1, const float* __restrict__ B1, int ldb1, int K1,
                                              const float* __restrict__ At2, int lda2, const float* __restrict__ B2, int ldb2, int K2,
                                              int M4, int N4, F&& emit) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  for (int m0 = ty * 4; m0 < M4; m0 += 64)
    for (int n0 = tx * 4; n0 < N4; n0 += 64) {
      float a1[4][4], a2[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) a1[i][j] = a2[i][j] = 0.f;
#pragma unroll 4
      for (int k = 0; k < K1; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(At1 + (size_t)k * lda1 + m0);
        const float4 b = *reinterpret_cast<const float4*>(B1 + (size_t)k * ldb1 + n0);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) a1[i][j] = fmaf(av[i], bv[j], a1[i][j]);
      }
#pragma unroll 4
      for (int k = 0; k < K2; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(At2 + (size_t)k * lda2 + m0);
        const float4 b = *reinterpret_cast<const float4*>(B2 + (size_t)k * ldb2 + n0);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) a2[i][j] = fmaf(av[i], bv[j], a2[i][j]);
      }
      emit(m0, n0, a1, a2);
    }
}

// scratch U: [S, max_pieces, heads, D * E]
template <typename T>
__global__ void __launch_bounds__(256) retention_piece_kernel(const T* __restrict__ proj, int row, int k_off, int v_off,
                                                              const float* __restrict__ decay, float kscale, float* __restrict__ U,
                                                              const int* __restrict__ cu_seqlens, int heads, int D, int E,
                                                              int max_pieces) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x, hd = blockIdx.y, s = blockIdx.z, tid = threadIdx.x;
  const int t0 = cu_seqlens[s] + p * RC, n = min(cu_seqlens[s + 1] - t0, RC);
  if (n <= 0) return;
  const int D4 = up4(D), E4 = up4(E);
  float* Kw = sm;                     // [RC][D4]: k_j * kscale * decay^(n-1-j)
  float* V = Kw + RC * D4;            // [RC][E4]
  const float l2 = log2f(decay[hd]);
  for (int i = tid; i < RC * D4; i += 256) {
    const int j = i / D4, d = i % D4;
    Kw[i] = (j < n && d < D) ? to_f32(proj[(size_t)(t0 + j) * row + k_off + hd * D + d]) * kscale * exp2f(l2 * (float)(n - 1 - j)) : 0.f;
  }
  for (int i = tid; i < RC * E4; i += 256) {
    const int j = i / E4, e = i % E4;
    V[i] = (j < n && e < E) ? to_f32(proj[(size_t)(t0 + j) * row + v_off + hd * E + e]) : 0.f;
  }
  __syncthreads();
  float* u = U + (((size_t)s * max_pieces + p) * heads + hd) * D * E;
  tile_product2(Kw, D4, V, E4, n, Kw, D4, V, E4, 0, D4, E4, [&](int m0, int n0, float (&a1)[4][4], float (&a2)[4][4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (m0 + i < D && n0 + j < E) u[(size_t)(m0 + i) * E + n0 + j] = a1[i][j];
  });
}

__global__ void __launch_bounds__(256) retention_carry_kernel(float* __restrict__ U, float* __restrict__ state,
                                                              const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                                                              const int* __restrict__ seq_slots, int heads, int DE, int max_pieces) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x / heads, hd = blockIdx.x % heads, i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= DE) return;
  const int n = cu_seqlens[s + 1] - cu_seqlens[s];
  const int pieces = (n + RC - 1) / RC;
  const float l2 = log2f(decay[hd]);
  float* sp = state + ((size_t)seq_slots[s] * heads + hd) * DE + i;
  float S = *sp;
  const float full = exp2f(l2 * (float)RC);
  for (int p0 = 0; p0 < pieces; p0 += 8) {                 // eight pieces' sums on the way at once, then the chain
    float add[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) add[k] = U[(((size_t)s * max_pieces + min(p0 + k, pieces - 1)) * heads + hd) * DE + i];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (p0 + k < pieces) {
        const int p = p0 + k;
        U[(((size_t)s * max_pieces + p) * heads + hd) * DE + i] = S;
        S = fmaf(n - p * RC >= RC ? full : exp2f(l2 * (float)(n - p * RC)), S, add[k]);
      }
  }
  *sp = S;
}

// Where the apply kernel's arrays lie in shared memory (in floats).  The keys' tile is dead once the scores are made, so the
// piece's begin state takes its place; and where a thread has at most one tile of outputs (value heads of up to 64) they
// wait in registers until the queries' tile is dead too and take its place: two blocks then fit an SM at 128 x 64 heads.
struct RetLayout { int qt, ks, v, wt, o, pw, total, o_alias; };
__host__ __device__ static inline RetLayout ret_layout(int D, int E) {
  const int E4 = up4(E), LT = RC + 4;
  RetLayout L;
  L.qt = 0;
  L.ks = D * LT;
  L.v = L.ks + (D * LT > D * E4 ? D * LT : D * E4);
  L.wt = L.v + RC * E4;
  int end = L.wt + RC * LT;
  L.o_alias = (E4 <= 64 && RC * E4 <= D * LT) ? 1 : 0;
  if (L.o_alias) {
    L.o = L.qt;
  } else {
    L.o = end;
    end += RC * E4;
  }
  L.pw = end;
  L.total = end + RC + 4;
  return L;
}

template <typename T>
__global__ void __launch_bounds__(256) retention_apply_kernel(const T* __restrict__ proj, int row, int q_off, int k_off, int v_off,
                                                              int g_off, const float* __restrict__ decay, float kscale, float eps,
                                                              int unit_norm, float out_scale, const float* __restrict__ U,
                                                              T* __restrict__ out, int out_stride, const int* __restrict__ cu_seqlens,
                                                              int heads, int D, int E, int max_pieces) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x, hd = blockIdx.y, s = blockIdx.z, tid = threadIdx.x;
  const int t0 = cu_seqlens[s] + p * RC, n = min(cu_seqlens[s + 1] - t0, RC);
  if (n <= 0) return;
  const int E4 = up4(E);
  constexpr int LT = RC + 4;          // leading size of the transposed arrays: their stores spread over banks
  const RetLayout L = ret_layout(D, E);
  float* Qt = sm + L.qt;              // [D][LT]   Qt[d][i] = q_i[d]
  float* Kt = sm + L.ks;              // [D][LT]   Kt[d][j] = k_j[d] * kscale; then
  float* Sb = sm + L.ks;              // [D][E4]   the state at the piece's begin
  float* V = sm + L.v;                // [RC][E4]
  float* Wt = sm + L.wt;              // [RC][LT]  Wt[j][i] = decay^(i-j) (q_i . k_j) for j <= i, else 0
  float* O = sm + L.o;                // [RC][E4]
  float* pw = sm + L.pw;              // [RC + 1]  decay^n
  const float l2 = log2f(decay[hd]);
  for (int i = tid; i <= RC; i += 256) pw[i] = exp2f(l2 * (float)i);
  for (int i = tid; i < RC * D; i += 256) {
    const int j = i / D, d = i % D;
    const bool ok = j < n;
    Qt[(size_t)d * LT + j] = ok ? to_f32(proj[(size_t)(t0 + j) * row + q_off + hd * D + d]) : 0.f;
    Kt[(size_t)d * LT + j] = ok ? to_f32(proj[(size_t)(t0 + j) * row + k_off + hd * D + d]) * kscale : 0.f;
  }
  for (int i = tid; i < D * 4; i += 256) {            // the padding columns RC .. RC+3 of both
    Qt[(size_t)(i / 4) * LT + RC + (i % 4)] = 0.f;
    Kt[(size_t)(i / 4) * LT + RC + (i % 4)] = 0.f;
  }
  for (int i = tid; i < RC * E4; i += 256) {
    const int j = i / E4, e = i % E4;
    V[i] = (j < n && e < E) ? to_f32(proj[(size_t)(t0 + j) * row + v_off + hd * E + e]) : 0.f;
  }
  __syncthreads();
  // Wt[j][i]: the product over d with m = j and n = i
  tile_product2(Kt, LT, Qt, LT, D, Kt, LT, Qt, LT, 0, RC, RC, [&](int m0, int n0, float (&a1)[4][4], float (&a2)[4][4]) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int j = m0 + a, i = n0 + b;
        Wt[j * LT + i] = (i >= j) ? a1[a][b] * pw[i - j] : 0.f;
      }
  });
  __syncthreads();
  const float* u = U + (((size_t)s * max_pieces + p) * heads + hd) * D * E;
  for (int i = tid; i < D * E4; i += 256) {           // over the keys' tile
    const int d = i / E4, e = i % E4;
    Sb[i] = e < E ? u[(size_t)d * E + e] : 0.f;
  }
  __syncthreads();
  // O[i][e] = sum_j Wt[j][i] V[j][e] + decay^(i+1) sum_d Qt[d][i] Sb[d][e]
  float held[4][4];
  int held_m = -1, held_n = 0;
  tile_product2(Wt, LT, V, E4, n, Qt, LT, Sb, E4, D, RC, E4, [&](int m0, int n0, float (&a1)[4][4], float (&a2)[4][4]) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float x = fmaf(pw[m0 + a + 1], a2[a][b], a1[a][b]);
        if (L.o_alias) held[a][b] = x;
        else O[(m0 + a) * E4 + n0 + b] = x;
      }
    held_m = m0;
    held_n = n0;
  });
  if (L.o_alias) {                                     // the outputs take the queries' place once every thread is done with it
    __syncthreads();
    if (held_m >= 0) {
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) O[(held_m + a) * E4 + held_n + b] = held[a][b];
    }
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int i = warp; i < n; i += 8) {
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) ss += O[i * E4 + e] * O[i * E4 + e];
    const float inv = unit_norm ? rsqrtf(warp_sum(ss) / (float)E + eps) : 1.f;
    const T* r = proj + (size_t)(t0 + i) * row;
    for (int e = lane; e < E; e += 32) {
      float x = O[i * E4 + e] * inv;
      if (g_off >= 0) x *= silu_f32(to_f32(r[g_off + hd * E + e]));
      out[(size_t)(t0 + i) * out_stride + hd * E + e] = from_f32<T>(x * out_scale);
    }
  }
}

static size_t retention_apply_smem(int D, int E) { return (size_t)ret_layout(D, E).total * sizeof(float); }
// can the long-portion form run for these sizes?  (its tiles have to fit an SM's shared memory)
extern "C" int sx_retention_pieces_fit(int D, int E) { return retention_apply_smem(D, E) <= 200 * 1024 ? 1 : 0; }
extern "C" int sx_retention_piece_tokens() { return RC; }

template <typename T>
static int retention_pieces_launch(const void* proj, int row, int q_off, int k_off, int v_off, int g_off, const float* decay,
                                   float kscale, float eps, int unit_norm, float out_scale, float* state, void* out,
                                   int out_stride, float* scratch, const int* cu_seqlens, const int* seq_slots, int S, int heads,
                                   int D, int E, int max_new, cudaStream_t stream) {
  const int max_pieces = (max_new + RC - 1) / RC;
  const size_t smem1 = ((size_t)RC * up4(D) + (size_t)RC * up4(E)) * sizeof(float);
  const size_t smem3 = retention_apply_smem(D, E);
  cudaError_t ce = cudaFuncSetAttribute(retention_piece_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
  if (ce != cudaSuccess) return (int)ce;
  ce = cudaFuncSetAttribute(retention_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
  if (ce != cudaSuccess) return (int)ce;
  const dim3 grid(max_pieces, heads, S);
  int e = sx_launch(retention_piece_kernel<T>, grid, dim3(256), smem1, stream, (const T*)proj, row, k_off, v_off, decay, kscale,
                    scratch, cu_seqlens, heads, D, E, max_pieces);
  if (e) return e;
  e = sx_launch(retention_carry_kernel, dim3(S * heads, (D * E + 255) / 256), dim3(256), 0, stream, scratch, state, decay, cu_seqlens,
                seq_slots, heads, D * E, max_pieces);
  if (e) return e;
  return sx_launch(retention_apply_kernel<T>, grid, dim3(256), smem3, stream, (const T*)proj, row, q_off, k_off, v_off, g_off, decay,
                   kscale, eps, unit_norm, out_scale, (const float*)scratch, (T*)out, out_stride, cu_seqlens, heads, D, E, max_pieces);
}

// mode 0: one block a (sequence, head) walks the tokens;  mode 1: single-token steps (row t is sequence t);
// mode 2: pieces (scratch float32 [S, ceil(max_new / 64), heads, D * E])
extern "C" int sx_retention_any(const void* proj, int row, int q_off, int k_off, int v_off, int g_off, const float* decay,
                                float kscale, float eps, int unit_norm, float out_scale, float* state, void* out, int out_stride,
                                float* scratch, const int* cu_seqlens, const int* seq_slots, int S, int heads, int D, int E,
                                int max_new, int mode, int dt, cudaStream_t stream) {
  if (S <= 0 || heads <= 0) return 0;
  if (D <= 0 || E <= 0 || E > 1024 || heads > 65535 || S > 65535) return SX_ERR_SIZE;
  if (mode == 2) {
    if (!scratch || !sx_retention_pieces_fit(D, E)) return SX_ERR_SIZE;
    if (dt == SX_F32)
      return retention_pieces_launch<float>(proj, row, q_off, k_off, v_off, g_off, decay, kscale, eps, unit_norm, out_scale, state, out,
                                            out_stride, scratch, cu_seqlens, seq_slots, S, heads, D, E, max_new, stream);
    if (dt == SX_BF16)
      return retention_pieces_launch<bf16>(proj, row, q_off, k_off, v_off, g_off, decay, kscale, eps, unit_norm, out_scale, state, out,
                                           out_stride, scratch, cu_seqlens, seq_slots, S, heads, D, E, max_new, stream);
    return SX_ERR_DTYPE;
  }
  if (mode == 1) {
    const int threads = E <= 256 ? 256 : (E <= 512 ? 512 : 1024);
    const int G = threads / E;
    const size_t smem = ((size_t)2 * D + (size_t)G * E) * sizeof(float);
    if (smem > 48 * 1024) return SX_ERR_SIZE;
    if (dt == SX_F32)
      return sx_launch(retention_step_kernel<float>, dim3(S, heads), dim3(threads), smem, stream, (const float*)proj, row, q_off, k_off,
                       v_off, g_off, decay, kscale, eps, unit_norm, out_scale, state, (float*)out, out_stride, seq_slots, heads, D, E);
    if (dt == SX_BF16)
      return sx_launch(retention_step_kernel<bf16>, dim3(S, heads), dim3(threads), smem, stream, (const bf16*)proj, row, q_off, k_off,
                       v_off, g_off, decay, kscale, eps, unit_norm, out_scale, state, (bf16*)out, out_stride, seq_slots, heads, D, E);
    return SX_ERR_DTYPE;
  }
  return sx_retention(proj, row, q_off, k_off, v_off, g_off, decay, kscale, eps, unit_norm, out_scale, state, out, out_stride,
                      cu_seqlens, seq_slots, S, heads, D, E, dt, stream);
}

// ---------------------------------------------------------------------------------------
// Capped gated activation of a stacked gate/up product gu [T, 2I]:
//   g = min(gu[t, i], limit),  u = clamp(gu[t, I + i], -limit, limit),  out = g * sigmoid(alpha g) * (u + 1)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void capped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, float alpha, float limit, int form, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  if (form == SX_GATE_GELU_TANH) {          // the tanh form of GELU of the gate, times up (precise functions: the 32-bit path)
    const float z = to_f32(gu[t * 2 * I + i]), u = to_f32(gu[t * 2 * I + I + i]);
    out[idx] = from_f32<T>(0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * u);
    return;
  }
  const float g = fminf(to_f32(gu[t * 2 * I + i]), limit);
  const float u = fminf(fmaxf(to_f32(gu[t * 2 * I + I + i]), -limit), limit);
  out[idx] = from_f32<T>(g * sigmoid_f32(alpha * g) * (u + 1.f));
}
extern "C" int sx_capped_glu(const void* gu, void* out, int n_tokens, int I, float alpha, float limit, int form, int dt, cudaStream_t stream) {
  const size_t n = (size_t)n_tokens * I;
  if (n == 0) return 0;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (dt == SX_F32) return sx_launch(capped_glu_kernel<float>, grid, dim3(256), 0, stream, (const float*)gu, (float*)out, I, alpha, limit, form, n);
  if (dt == SX_BF16) return sx_launch(capped_glu_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, I, alpha, limit, form, n);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// h[t, c] += delta[t, c] + rows[t, c] + vec[c]   (each of the three optional; h, rows and vec 32-bit)
// ---------------------------------------------------------------------------------------
template <typename TD>
__global__ void stream_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ rows,
                                  const float* __restrict__ vec, int H, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  float v = h[idx];
  if (delta) v += to_f32(delta[idx]);
  if (rows) v += rows[idx];
  if (vec) v += vec[idx % H];
  h[idx] = v;
}
extern "C" int sx_stream_add(float* h, const void* delta, int delta_dt, const float* rows, const float* vec, int n_tokens, int H,
                             cudaStream_t stream) {
  const size_t n = (size_t)n_tokens * H;
  if (n == 0) return 0;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (delta_dt == SX_F32) return sx_launch(stream_add_kernel<float>, grid, dim3(256), 0, stream, h, (const float*)delta, rows, vec, H, n);
  if (delta_dt == SX_BF16) return sx_launch(stream_add_kernel<bf16>, grid, dim3(256), 0, stream, h, (const bf16*)delta, rows, vec, H, n);
  return SX_ERR_DTYPE;
}
