// A mixture of gated feed-forward experts (sm_100a), float32 and bfloat16; router, softmax and weights are 32-bit.
//
//   moe_route_kernel   one block a token (four in prompt steps): logits z_e = Wr[e] . x in 32-bit (Wr float32, x widened), softmax over ALL
//                      experts (or a sigmoid each), the `top` largest choice values (ties: the lower index; optionally
//                      with a correction per expert and only within the best groups, see RouteMode), weights = score /
//                      (sum of the chosen + sum_eps) * scale, or score * scale  -> ids [T, top], weights [T, top]
//   moe_sort_kernel    one block: the T * top (token, choice) pairs sorted by expert: offsets [E + 1], order [T * top]
//                      (sorted place -> pair), place [T * top] (pair -> sorted place).  The order inside an expert's
//                      group is whatever the atomics give; no result depends on it (each row is computed alone).
//   moe_gemm_kernel    grouped product: tile i of the grid's y axis belongs to the expert whose rows hold it (a block
//                      finds it from `offsets`; tiles beyond the last return).  GATE_UP: rows are gathered from x by
//                      pair / top, the expert's [gate; up] matrix gives two accumulators and the result is
//                      silu(gate) * up  [T * top, ff] in sorted order; else rows are read in sorted order and the
//                      result is the plain product [T * top, N].  64x64x16 tiles, 4x4 results a thread, 32-bit FFMA
//                      (float32, and bfloat16 with K % 8 != 0).
//   moe_mma_kernel     the same product for bfloat16 on the tensor cores (see there).
//   moe_combine_kernel out[t] = sum_j weights[t, j] * y[place[t * top + j]], the choices in their order.
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024

#define MOE_ROUTE_THREADS 512

// How the router turns logits into choices and weights:
//   sigmoid     0: scores = softmax over all experts; 1: scores = sigmoid(logit), each expert alone
//   correction  float32 [E] or null: added to the scores for the CHOICE only (the weights use the scores without it)
//   groups, keep  the experts form `groups` equal groups of neighbours; a group's value is the sum of its two largest
//               choice values (of its one, if a group is one expert) and only experts of the `keep` best groups (ties:
//               the lower group) can be chosen; groups <= 1: every expert can
//   renorm      1: weights = score / (sum of the chosen scores + sum_eps) * scale; 0: weights = score * scale
struct RouteMode { int sigmoid; const float* correction; int groups, keep, renorm; };

// TB tokens a block: a warp reads an expert's router row once for all of them; warp i then chooses for token i
template <typename T, int TB>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS) moe_route_kernel(const T* __restrict__ x, const float* __restrict__ wr, int n_tokens,
                                                                       int W, int E, int top, float scale, float sum_eps,
                                                                       int* __restrict__ ids, float* __restrict__ weights,
                                                                       const RouteMode mode) {
  extern __shared__ __align__(16) float sm[];
  float* xs = sm;                 // TB * W
  float* zs = sm + TB * W;        // TB * E: scores
  float* cs = zs + TB * E;        // TB * E: choice values
  float* gs = cs + TB * E;        // TB * groups: the groups' values
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.x * TB, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = min(TB, n_tokens - t0);
  for (int i = tid; i < TB * W; i += MOE_ROUTE_THREADS) {
    const int tt = i / W;
    xs[i] = tt < nt ? to_f32(x[(size_t)t0 * W + i]) : 0.f;
  }
  __syncthreads();
  for (int e = warp; e < E; e += MOE_ROUTE_THREADS / 32) {
    const float* w = wr + (size_t)e * W;
    float d[TB];
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) d[tt] = 0.f;
    if ((W & 3) == 0 && ((uintptr_t)wr & 15) == 0) {          // 16 bytes a load, four loads on the way
#pragma unroll 4
      for (int i = lane * 4; i < W; i += 128) {
        const float4 w4 = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) {
          const float4 x4 = *reinterpret_cast<const float4*>(xs + tt * W + i);
          d[tt] = fmaf(x4.x, w4.x, fmaf(x4.y, w4.y, fmaf(x4.z, w4.z, fmaf(x4.w, w4.w, d[tt]))));
        }
      }
    } else {
      for (int i = lane; i < W; i += 32) {
        const float wi = w[i];
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) d[tt] = fmaf(xs[tt * W + i], wi, d[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < TB; ++tt) {
      const float v = warp_sum(d[tt]);
      if (lane == 0) zs[tt * E + e] = v;
    }
  }
  __syncthreads();
  if (warp >= nt) return;
  const int t = t0 + warp;
  float* z = zs + warp * E;
  float* c = cs + warp * E;
  float sum = 1.f;
  if (mode.sigmoid) {
    for (int e = lane; e < E; e += 32) z[e] = 1.f / (1.f + expf(-z[e]));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - mx); z[e] = p; sum += p; }
    sum = warp_sum(sum);
  }
  for (int e = lane; e < E; e += 32) c[e] = z[e] + (mode.correction ? mode.correction[e] : 0.f);
  __syncwarp();
  if (mode.groups > 1) {
    // a lane a group: the sum of its two largest choice values; then the `keep` best groups stay, by rank
    float* g = gs + warp * mode.groups;
    const int size = E / mode.groups;
    for (int gi = lane; gi < mode.groups; gi += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int e = gi * size; e < (gi + 1) * size; ++e) {
        const float v = c[e];
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
      }
      g[gi] = size > 1 ? a + b : a;
    }
    __syncwarp();
    for (int gi = lane; gi < mode.groups; gi += 32) {
      const float v = g[gi];
      int rank = 0;                                  // how many groups come before this one
      for (int o = 0; o < mode.groups; ++o) rank += (g[o] > v || (g[o] == v && o < gi)) ? 1 : 0;
      if (rank >= mode.keep)
        for (int e = gi * size; e < (gi + 1) * size; ++e) c[e] = -INFINITY;
    }
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float p = c[e];
      if (p > best) { best = p; bi = e; }       // a lane walks upwards: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= E) bi = 0;                           // nothing left to choose (NaN logits): keep the index in range
    const float s = z[bi] / sum;
    chosen_sum += s;
    if (lane == 0) {
      ids[(size_t)t * top + j] = bi;
      weights[(size_t)t * top + j] = s;
    }
    __syncwarp();
    if (lane == 0) c[bi] = -INFINITY;              // taken
    __syncwarp();
  }
  const float f = mode.renorm ? scale / (chosen_sum + sum_eps) : scale;
  for (int j = lane; j < top; j += 32) weights[(size_t)t * top + j] *= f;
}

template <typename T, int TB>
static int moe_route_launch(const void* x, const float* wr, int T_, int W, int E, int top, float scale, float sum_eps, int* ids,
                            float* weights, const RouteMode mode, cudaStream_t stream) {
  const size_t smem = (size_t)TB * (W + 2 * E + (mode.groups > 1 ? mode.groups : 0)) * sizeof(float);
  if (smem > 160 * 1024) return SX_ERR_SIZE;
  if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<T, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return sx_launch(moe_route_kernel<T, TB>, dim3((T_ + TB - 1) / TB), dim3(MOE_ROUTE_THREADS), smem, stream, (const T*)x, wr, T_, W, E,
                   top, scale, sum_eps, ids, weights, mode);
}

extern "C" int sx_moe_route(const void* x, const float* wr, int T, int W, int E, int top, float scale, float sum_eps,
                            int* ids, float* weights, int sigmoid, const float* correction, int groups, int keep, int renorm,
                            int dt, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || W <= 0) return SX_ERR_SIZE;
  if (groups > 1 && (E % groups || keep <= 0 || keep > groups || top > keep * (E / groups))) return SX_ERR_SIZE;
  const RouteMode mode = {sigmoid, correction, groups, keep, renorm};
  // prompt steps: four tokens a block share every router row they read (where that fits shared memory)
  const bool four = T >= 256 && (size_t)4 * (W + 2 * E + (groups > 1 ? groups : 0)) * sizeof(float) <= 160 * 1024;
  if (dt == SX_F32)
    return four ? moe_route_launch<float, 4>(x, wr, T, W, E, top, scale, sum_eps, ids, weights, mode, stream)
                : moe_route_launch<float, 1>(x, wr, T, W, E, top, scale, sum_eps, ids, weights, mode, stream);
  if (dt == SX_BF16)
    return four ? moe_route_launch<bf16, 4>(x, wr, T, W, E, top, scale, sum_eps, ids, weights, mode, stream)
                : moe_route_launch<bf16, 1>(x, wr, T, W, E, top, scale, sum_eps, ids, weights, mode, stream);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ offsets,
                                                        int* __restrict__ order, int* __restrict__ place) {
  __shared__ int count[MOE_MAX_EXPERTS];
  __shared__ int start[MOE_MAX_EXPERTS + 1];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) count[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (tid == 0) {
    int s = 0;
    for (int e = 0; e < E; ++e) { start[e] = s; s += count[e]; }
    start[E] = s;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += 1024) offsets[e] = start[e];
  for (int e = tid; e < E; e += 1024) count[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    const int p = start[e] + atomicAdd(&count[e], 1);
    order[p] = i;
    place[i] = p;
  }
}

extern "C" int sx_moe_sort(const int* ids, int n, int E, int* offsets, int* order, int* place, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS) return SX_ERR_SIZE;
  return sx_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, ids, n, E, offsets, order, place);
}

// ---------------------------------------------------------------------------------------------------------------
// the experts' gated activation (the library's value, see common.cuh), with precise exponentials: this file also
// serves the 32-bit path
__device__ __forceinline__ float moe_gate(float g, float u, const GateAct a) {
  if (a.form == SX_GATE_GELU_TANH) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (a.limit > 0.f) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.f + expf(-a.alpha * g)) * (u + 1.f);
  }
  return g / (1.f + expf(-g)) * u;
}

template <typename TA, typename TW, typename TC, bool GATE_UP>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ Wt, TC* __restrict__ C,
                                                       const int* __restrict__ offsets, const int* __restrict__ order,
                                                       int E, int N, int K, int top, const GateAct act) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[GATE_UP ? BK : 1][BN + 4];
  __shared__ int src[BM];
  __shared__ int which[3];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  if (tid == 0) {
    // the tile's expert and first row: tiles are counted expert by expert
    int tile = blockIdx.y, e = 0, r0 = -1;
    for (; e < E; ++e) {
      const int n_e = offsets[e + 1] - offsets[e];
      const int tiles = (n_e + BM - 1) / BM;
      if (tile < tiles) { r0 = offsets[e] + tile * BM; break; }
      tile -= tiles;
    }
    which[0] = e; which[1] = r0; which[2] = r0 >= 0 ? min(BM, offsets[e + 1] - r0) : 0;
  }
  __syncthreads();
  const int e = which[0], r0 = which[1], nr = which[2];
  if (r0 < 0) return;
  if (tid < BM) src[tid] = tid < nr ? (GATE_UP ? order[r0 + tid] / top : r0 + tid) : -1;
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * BN;
  const int NW = GATE_UP ? 2 * N : N;         // rows of an expert's matrix
  const TW* We = Wt + (size_t)e * NW * K;
  float acc[4][4], acu[GATE_UP ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GATE_UP) acu[i][j] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = idx & 15;
      const int k = k0 + c;
      const int m = src[r], n = n0 + r;
      As[c][r] = (m >= 0 && k < K) ? to_f32(A[(size_t)m * K + k]) : 0.f;
      Ws[c][r] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
      if (GATE_UP) Us[c][r] = (n < N && k < K) ? to_f32(We[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = Ws[kk][tx * 4 + j]; if (GATE_UP) u[j] = Us[kk][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATE_UP) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= nr) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)(r0 + r) * N + n] = from_f32<TC>(GATE_UP ? moe_gate(acc[i][j], acu[i][j], act) : acc[i][j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same grouped product for bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulation): a block of 8
// warps (2 along the rows x 4 along the columns) owns 64 rows x 128 matrix rows; with GATE_UP these are 64 gate rows
// and the 64 up rows of the same outputs, so a thread holds gate and up of one place and the activation needs no
// exchange.  Rows of x (gathered through `order`) and of the expert's matrix come by cp.async, 16 bytes a copy,
// through a ring of stages of 64 k each (128 bytes of a row a stage); fragments by ldmatrix from rows padded
// to 144 bytes.  With a few
// rows per expert (single-token steps) a block still streams its 128 matrix rows once: the kernel is then bound by
// the experts' weights, which each active expert's blocks read exactly once.  K % 8 == 0.
// ---------------------------------------------------------------------------------------------------------------
#define MM_BN 128
#define MM_BK 64
#define MM_LD 72             // elements of a staged row (64 + 8 of padding)
// rows a block (BM) and stages of its ring: 64 rows with 4 stages, or, for steps whose experts get a handful of rows
// each, 16 rows with 5 stages; two blocks an SM either way (a gate/up product of 152 blocks then runs in one round of
// the 148 SMs; with one block an SM the last 4 blocks made a second round), eight stages of 18 KB of weights on the way
template <int BM> struct MmShape {
  static constexpr int STAGES = BM == 64 ? 4 : 5;
  static constexpr int WARPS_M = BM == 64 ? 2 : 1;
  static constexpr int WARPS_N = 8 / WARPS_M;
  static constexpr int MI = BM / (16 * WARPS_M);                    // m16 tiles a warp
  static constexpr int NT = MM_BN / WARPS_N / 8;                     // n8 tiles a warp: 4 or 2
  static constexpr size_t SMEM = (size_t)STAGES * (BM + MM_BN) * MM_LD * sizeof(bf16);
};

__device__ __forceinline__ void mm_cp16(void* smem, const void* gmem, bool ok) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem);
  const int n = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void mm_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void mm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mm_ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TC, bool GATE_UP, int BM>
__global__ void __launch_bounds__(256) moe_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ Wt, TC* __restrict__ C,
                                                      const int* __restrict__ offsets, const int* __restrict__ order,
                                                      int E, int N, int K, int top, const GateAct act) {
  using Sh = MmShape<BM>;
  constexpr int STAGES = Sh::STAGES, MI = Sh::MI, NT = Sh::NT;
  extern __shared__ __align__(16) unsigned char mm_smem[];
  bf16* As = (bf16*)mm_smem;                                        // STAGES * BM * MM_LD
  bf16* Ws = As + STAGES * BM * MM_LD;                              // STAGES * MM_BN * MM_LD
  __shared__ int src[BM];
  __shared__ int which[3];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    int tile = blockIdx.y, e = 0, r0 = -1;
    for (; e < E; ++e) {
      const int n_e = offsets[e + 1] - offsets[e];
      const int tiles = (n_e + BM - 1) / BM;
      if (tile < tiles) { r0 = offsets[e] + tile * BM; break; }
      tile -= tiles;
    }
    which[0] = e; which[1] = r0; which[2] = r0 >= 0 ? min(BM, offsets[e + 1] - r0) : 0;
  }
  __syncthreads();
  const int e = which[0], r0 = which[1], nr = which[2];
  if (r0 < 0) return;
  if (tid < BM) src[tid] = tid < nr ? (GATE_UP ? order[r0 + tid] / top : r0 + tid) : -1;
  __syncthreads();
  constexpr int NOUT = GATE_UP ? MM_BN / 2 : MM_BN;                 // output columns of a block
  const int n0 = blockIdx.x * NOUT;
  const bf16* We = Wt + (size_t)e * (GATE_UP ? 2 : 1) * N * K;
  // what this thread copies each stage: 16-byte piece a_ch of (up to) two rows of x and of four rows of the matrix
  constexpr int A_COPIES = (BM * 8 + 255) / 256;
  const int a_ch = tid & 7;
  const bf16* a_src[A_COPIES];
  bool a_ok[A_COPIES];
#pragma unroll
  for (int i = 0; i < A_COPIES; ++i) {
    const int r = (tid + i * 256) >> 3;
    a_ok[i] = r < BM && src[r < BM ? r : 0] >= 0;
    a_src[i] = A + (size_t)(a_ok[i] ? src[r] : 0) * K + a_ch * 8;
  }
  const bf16* w_src[4];
  bool w_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (tid + i * 256) >> 3;                              // row of the staged tile
    int n;                                                           // row of the expert's matrix
    bool ok;
    if (GATE_UP) { const int c = n0 + (r & 63); ok = c < N; n = (r < 64 ? 0 : N) + c; }
    else { n = n0 + r; ok = n < N; }
    w_ok[i] = ok;
    w_src[i] = We + (size_t)(ok ? n : 0) * K + a_ch * 8;
  }
  const int nk = (K + MM_BK - 1) / MM_BK;
  auto load = [&](int kt, int stage) {
    const int k0 = kt * MM_BK;
    const bool kin = k0 + a_ch * 8 < K;
#pragma unroll
    for (int i = 0; i < A_COPIES; ++i) {
      const int r = (tid + i * 256) >> 3;
      if (r < BM) mm_cp16(As + ((size_t)stage * BM + r) * MM_LD + a_ch * 8, a_src[i] + k0, a_ok[i] && kin);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      mm_cp16(Ws + ((size_t)stage * MM_BN + ((tid + i * 256) >> 3)) * MM_LD + a_ch * 8, w_src[i] + k0, w_ok[i] && kin);
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    mm_commit();
  }
  const int wm = warp / Sh::WARPS_N, wn = warp % Sh::WARPS_N;       // a warp: MI m16 tiles x NT n8 tiles
  float acc[MI][NT][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[i][j][x] = 0.f;
  for (int kt = 0; kt < nk; ++kt) {
    mm_wait<STAGES - 2>();
    __syncthreads();                                                 // stage kt has landed; stage kt - 1 is read out
    if (kt + STAGES - 1 < nk) load(kt + STAGES - 1, (kt + STAGES - 1) % STAGES);
    mm_commit();
    const bf16* as = As + (size_t)(kt % STAGES) * BM * MM_LD;
    const bf16* ws = Ws + (size_t)(kt % STAGES) * MM_BN * MM_LD;
#pragma unroll
    for (int kk = 0; kk < MM_BK / 16; ++kk) {
      uint32_t af[MI][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        mm_ldsm4(af[mi][0], af[mi][1], af[mi][2], af[mi][3],
                 as + (size_t)(wm * MI * 16 + mi * 16 + (lane & 15)) * MM_LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int pair = 0; pair < NT / 2; ++pair) {                    // two n8 tiles a load
        // the staged row of this lane's address.  GATE_UP: a warp's gate tiles first, then its up tiles (staged rows
        // 64 ..): with four tiles a warp pair 0 = gate, pair 1 = up; with two the one load takes a gate and an up tile
        const int sub = lane >> 4;
        int nb;
        if (!GATE_UP) nb = wn * NT * 8 + pair * 16 + sub * 8;
        else if (NT == 4) nb = pair * 64 + wn * 16 + sub * 8;
        else nb = sub * 64 + wn * 8;
        uint32_t b0, b1, b2, b3;
        mm_ldsm4(b0, b1, b2, b3, ws + (size_t)(nb + (lane & 7)) * MM_LD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          mm_mma(acc[mi][pair * 2], af[mi], b0, b1);
          mm_mma(acc[mi][pair * 2 + 1], af[mi], b2, b3);
        }
      }
    }
  }
  mm_wait<0>();
  const int row_in = lane >> 2, col_in = (lane & 3) * 2;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * MI * 16 + mi * 16 + half * 8 + row_in;
      if (r >= nr) continue;
      TC* crow = C + (size_t)(r0 + r) * N;
      if (GATE_UP) {
#pragma unroll
        for (int j = 0; j < NT / 2; ++j)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int n = n0 + wn * (NT / 2) * 8 + j * 8 + col_in + x;
            if (n < N) crow[n] = from_f32<TC>(moe_gate(acc[mi][j][half * 2 + x], acc[mi][NT / 2 + j][half * 2 + x], act));
          }
      } else {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int n = n0 + wn * NT * 8 + j * 8 + col_in + x;
            if (n < N) crow[n] = from_f32<TC>(acc[mi][j][half * 2 + x]);
          }
      }
    }
}

template <typename TC, bool GATE_UP, int BM>
static int moe_mma_launch(const void* A, const void* Wt, void* C, const int* offsets, const int* order, int rows, int E, int N,
                          int K, int top, cudaStream_t stream) {
  const size_t smem = MmShape<BM>::SMEM;
  static bool set = false;
  if (!set) {
    cudaError_t err = cudaFuncSetAttribute(moe_mma_kernel<TC, GATE_UP, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    set = true;
  }
  const int tiles = (rows + BM - 1) / BM + (E < rows ? E : rows);
  if (tiles > 65535) return SX_ERR_SIZE;
  const int nout = GATE_UP ? MM_BN / 2 : MM_BN;
  dim3 grid((N + nout - 1) / nout, tiles);
  return sx_launch(moe_mma_kernel<TC, GATE_UP, BM>, grid, dim3(256), smem, stream, (const bf16*)A, (const bf16*)Wt, (TC*)C, offsets,
                   order, E, N, K, top, g_sx_gate);
}

// up to this many (token, choice) rows a step, blocks of 16 rows with the deeper ring
#define MM_FEW_ROWS 64

// rows: T * top; the grid's y axis has room for every expert's last, partly filled tile
extern "C" int sx_moe_gemm(const void* A, const void* Wt, void* C, const int* offsets, const int* order, int rows, int E, int N,
                           int K, int top, int gate_up, int a_dt, int c_dt, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || N <= 0 || K <= 0) return SX_ERR_SIZE;
  const int tiles = (rows + 63) / 64 + (E < rows ? E : rows);
  if (tiles > 65535) return SX_ERR_SIZE;
  if (a_dt == SX_BF16 && K % 8 == 0 && ((uintptr_t)A | (uintptr_t)Wt) % 16 == 0) {       // the tensor cores
#define MM_GO(TC, GU)                                                                                               \
  return rows <= MM_FEW_ROWS ? moe_mma_launch<TC, GU, 16>(A, Wt, C, offsets, order, rows, E, N, K, top, stream)    \
                             : moe_mma_launch<TC, GU, 64>(A, Wt, C, offsets, order, rows, E, N, K, top, stream)
    if (gate_up && c_dt == SX_BF16) MM_GO(bf16, true);
    if (!gate_up && c_dt == SX_F32) MM_GO(float, false);
    if (!gate_up && c_dt == SX_BF16) MM_GO(bf16, false);
#undef MM_GO
  }
  dim3 grid((N + 63) / 64, tiles);
#define MOE_GO(TA, TC, GU) return sx_launch(moe_gemm_kernel<TA, TA, TC, GU>, grid, dim3(256), 0, stream, (const TA*)A, (const TA*)Wt, (TC*)C, offsets, order, E, N, K, top, g_sx_gate)
  if (gate_up) {
    if (a_dt == SX_F32 && c_dt == SX_F32) MOE_GO(float, float, true);
    if (a_dt == SX_BF16 && c_dt == SX_BF16) MOE_GO(bf16, bf16, true);
  } else {
    if (a_dt == SX_F32 && c_dt == SX_F32) MOE_GO(float, float, false);
    if (a_dt == SX_BF16 && c_dt == SX_F32) MOE_GO(bf16, float, false);
    if (a_dt == SX_BF16 && c_dt == SX_BF16) MOE_GO(bf16, bf16, false);
  }
#undef MOE_GO
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------------------------
template <typename TY, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   TO* __restrict__ out, int W, int top) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < top; ++j)
      s = fmaf(weights[(size_t)t * top + j], to_f32(y[(size_t)place[(size_t)t * top + j] * W + c]), s);
    out[(size_t)t * W + c] = from_f32<TO>(s);
  }
}

extern "C" int sx_moe_combine(const void* y, int y_dt, const int* place, const float* weights, void* out, int out_dt, int T,
                              int W, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (y_dt == SX_F32 && out_dt == SX_F32)
    return sx_launch(moe_combine_kernel<float, float>, dim3(T), dim3(256), 0, stream, (const float*)y, place, weights, (float*)out, W, top);
  if (y_dt == SX_F32 && out_dt == SX_BF16)
    return sx_launch(moe_combine_kernel<float, bf16>, dim3(T), dim3(256), 0, stream, (const float*)y, place, weights, (bf16*)out, W, top);
  if (y_dt == SX_BF16 && out_dt == SX_BF16)
    return sx_launch(moe_combine_kernel<bf16, bf16>, dim3(T), dim3(256), 0, stream, (const bf16*)y, place, weights, (bf16*)out, W, top);
  return SX_ERR_DTYPE;
}
