// Attention whose weights are a function of ALL heads' scores of a (query, key) pair, over the paged cache, in 32-bit
// FFMA (scores, their mixture over heads, the weights and the weighted sums of values never leave 32-bit):
//
//   s_g(i, j)  = (q_g(i) . k_kv(g)(j)) * scale                       for every query head g
//   s'_h(i, j) = sum_g talk[h, g] s_g(i, j)                          (talk null: s'_h = s_h)
//              + head_bias[h] + dist_bias[h, min(i - j, dist_n - 1)] (each null: not added)
//   weight     = sigmoid(s'_h)  (not normalised over keys)   or   softmax over the visible keys
//   o_h(i)     = sum_j weight_h(i, j) v_kv(h)(j)  [* gate[i, h]]
//
// Key j is visible to the query at position i iff j <= i and (window == 0 or j > i - window).
//
// heads_prepare_kernel makes q, k, v out of a float32 projection row [q heads | k heads | v heads | gates]: bias,
// optional RMS norm of every q and k head with a gain shared by the heads, optional rotation of NEIGHBOURING pairs
// (2i, 2i + 1) of the first rot_dims elements by position * inv_freq[i] with cos and sin times `mag`, optional blend of
// the values with those another layer made for the same token (v <- (1 - lam) v + lam v_first), cache write, and
// sigmoid of the gate columns.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_acc(float x) { return 1.f / (1.f + expf(-x)); }

// ---------------------------------------------------------------------------------------
// head preparation: grid (tokens, groups of four heads), a warp a head
// ---------------------------------------------------------------------------------------
struct PrepArgs {
  const float* proj; int row; const float* bias;
  void* q_out; void* k_pages; void* v_pages;
  const int* positions; const int* seq_of_token; const int* block_table; int maxp; int n_pages;
  int H, G, dim, vdim;
  const float* qn; const float* kn; float eps;
  const float* inv_freq; int rot_dims; float mag;
  const float* v_first_in; float* v_first_out; const float* lam;
  float* gate_out; int n_gate;
  int vec;        // every head is a multiple of four elements and every pointer 16-byte aligned: four elements a lane
};

__device__ __forceinline__ void prep_st4(float* p, float x, float y, float z, float w) {
  *reinterpret_cast<float4*>(p) = make_float4(x, y, z, w);
}
__device__ __forceinline__ void prep_st4(bf16* p, float x, float y, float z, float w) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(x, y), hi = __floats2bfloat162_rn(z, w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 prep_ld4(const float* p, const float* b) {
  float4 x = *reinterpret_cast<const float4*>(p);
  if (b) { const float4 y = *reinterpret_cast<const float4*>(b); x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
  return x;
}

template <typename T>
__global__ void __launch_bounds__(128) heads_prepare_kernel(const PrepArgs a) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = a.positions[t];
  const float* src_tok = a.proj + (size_t)t * a.row;
  const int s = a.seq_of_token[t];
  const int page = a.block_table[(size_t)s * a.maxp + (pos >> 6)];
  const bool page_ok = page >= 0 && page < a.n_pages;
  const int H = a.H, G = a.G, dim = a.dim, vdim = a.vdim;
  const int half = a.inv_freq ? a.rot_dims / 2 : 0;
  const float lam = (a.v_first_in && a.lam) ? *a.lam : 0.f;

  for (int head = blockIdx.y * 4 + warp; head < H + 2 * G; head += 4 * gridDim.y) {
    const bool is_q = head < H, is_k = !is_q && head < H + G;
    if (is_q || is_k) {
      const int col = head * dim;
      const float* src = src_tok + col;
      const float* bs = a.bias ? a.bias + col : nullptr;
      const float* gain = is_q ? a.qn : a.kn;
      T* dst;
      if (is_q) {
        dst = (T*)a.q_out + ((size_t)t * H + head) * dim;
      } else {
        if (!a.k_pages || !page_ok) continue;
        dst = (T*)a.k_pages + (((size_t)page * G + (head - H)) * SX_PAGE + (pos & 63)) * dim;
      }
      float inv = 1.f;
      if (a.vec) {
        // four elements a lane (two pairs of the rotation): 16-byte loads, 8- or 16-byte stores
        if (gain) {
          float ss = 0.f;
          for (int d = lane * 4; d < dim; d += 128) {
            const float4 x = prep_ld4(src + d, bs ? bs + d : nullptr);
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
          }
          inv = rsqrtf(warp_sum(ss) / (float)dim + a.eps);
        }
        for (int d = lane * 4; d < dim; d += 128) {
          float4 x = prep_ld4(src + d, bs ? bs + d : nullptr);
          if (gain) {
            const float4 gn = *reinterpret_cast<const float4*>(gain + d);
            x.x *= inv * gn.x; x.y *= inv * gn.y; x.z *= inv * gn.z; x.w *= inv * gn.w;
          }
          if (d < 2 * half) {
            float s0, c0, s1, c1;
            sincosf((float)pos * a.inv_freq[d >> 1], &s0, &c0);
            sincosf((float)pos * a.inv_freq[(d >> 1) + 1], &s1, &c1);
            s0 *= a.mag; c0 *= a.mag; s1 *= a.mag; c1 *= a.mag;
            x = make_float4(x.x * c0 - x.y * s0, x.y * c0 + x.x * s0, x.z * c1 - x.w * s1, x.w * c1 + x.z * s1);
          }
          prep_st4(dst + d, x.x, x.y, x.z, x.w);
        }
        continue;
      }
      if (gain) {
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) { const float x = src[d] + (bs ? bs[d] : 0.f); ss += x * x; }
        inv = rsqrtf(warp_sum(ss) / (float)dim + a.eps);
      }
      for (int i = lane; i < half; i += 32) {
        float u = src[2 * i] + (bs ? bs[2 * i] : 0.f), v = src[2 * i + 1] + (bs ? bs[2 * i + 1] : 0.f);
        if (gain) { u *= inv * gain[2 * i]; v *= inv * gain[2 * i + 1]; }
        float sn, cs;
        sincosf((float)pos * a.inv_freq[i], &sn, &cs);
        sn *= a.mag; cs *= a.mag;
        dst[2 * i] = from_f32<T>(u * cs - v * sn);
        dst[2 * i + 1] = from_f32<T>(v * cs + u * sn);
      }
      for (int d = 2 * half + lane; d < dim; d += 32) {
        float x = src[d] + (bs ? bs[d] : 0.f);
        if (gain) x *= inv * gain[d];
        dst[d] = from_f32<T>(x);
      }
    } else {
      const int c = head - H - G;
      const int col = (H + G) * dim + c * vdim;
      const float* src = src_tok + col;
      T* dst = (a.v_pages && page_ok) ? (T*)a.v_pages + (((size_t)page * G + c) * SX_PAGE + (pos & 63)) * vdim : nullptr;
      if (a.vec) {
        for (int d = lane * 4; d < vdim; d += 128) {
          float4 x = prep_ld4(src + d, a.bias ? a.bias + col + d : nullptr);
          const size_t vi = ((size_t)t * G + c) * vdim + d;
          if (a.v_first_in) {
            const float4 f = *reinterpret_cast<const float4*>(a.v_first_in + vi);
            x.x = (1.f - lam) * x.x + lam * f.x; x.y = (1.f - lam) * x.y + lam * f.y;
            x.z = (1.f - lam) * x.z + lam * f.z; x.w = (1.f - lam) * x.w + lam * f.w;
          }
          if (a.v_first_out) *reinterpret_cast<float4*>(a.v_first_out + vi) = x;
          if (dst) prep_st4(dst + d, x.x, x.y, x.z, x.w);
        }
        continue;
      }
      for (int d = lane; d < vdim; d += 32) {
        float x = src[d] + (a.bias ? a.bias[col + d] : 0.f);
        const size_t vi = ((size_t)t * G + c) * vdim + d;
        if (a.v_first_in) x = (1.f - lam) * x + lam * a.v_first_in[vi];
        if (a.v_first_out) a.v_first_out[vi] = x;
        if (dst) dst[d] = from_f32<T>(x);
      }
    }
  }
  if (a.gate_out && blockIdx.y == 0) {
    const int col = (H + G) * dim + G * vdim;
    for (int i = threadIdx.x; i < a.n_gate; i += blockDim.x)
      a.gate_out[(size_t)t * a.n_gate + i] = sigmoid_acc(src_tok[col + i] + (a.bias ? a.bias[col + i] : 0.f));
  }
}

extern "C" int sx_heads_prepare(const float* proj, int row, const float* bias, void* q_out, void* k_pages, void* v_pages,
                                const int* positions, const int* seq_of_token, const int* block_table, int maxp, int n_pages,
                                int n_tokens, int H, int G, int dim, int vdim, const float* qn, const float* kn, float eps,
                                const float* inv_freq, int rot_dims, float mag, const float* v_first_in, float* v_first_out,
                                const float* lam, float* gate_out, int n_gate, int dt, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > dim ||
      row < (H + G) * dim + G * vdim + n_gate)
    return SX_ERR_SIZE;
  PrepArgs a;
  a.proj = proj; a.row = row; a.bias = bias; a.q_out = q_out; a.k_pages = k_pages; a.v_pages = v_pages;
  a.positions = positions; a.seq_of_token = seq_of_token; a.block_table = block_table; a.maxp = maxp; a.n_pages = n_pages;
  a.H = H; a.G = G; a.dim = dim; a.vdim = vdim; a.qn = qn; a.kn = kn; a.eps = eps; a.inv_freq = inv_freq;
  a.rot_dims = rot_dims; a.mag = mag; a.v_first_in = v_first_in; a.v_first_out = v_first_out; a.lam = lam;
  a.gate_out = gate_out; a.n_gate = n_gate;
  a.vec = dim % 4 == 0 && vdim % 4 == 0 && rot_dims % 4 == 0 && row % 4 == 0 &&
          (((uintptr_t)proj | (uintptr_t)bias | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)qn |
            (uintptr_t)kn | (uintptr_t)v_first_in | (uintptr_t)v_first_out) & 15) == 0;
  // few tokens: a block for every four heads, so that a single token's heads spread over the GPU; many tokens: up to
  // four blocks a token, so that a warp walks a few heads one after the other, not a dozen
  const int groups = (H + 2 * G + 3) / 4;
  const dim3 grid(n_tokens, n_tokens >= 1024 ? (groups < 4 ? groups : 4) : (groups > 65535 ? 65535 : groups));
  if (dt == SX_F32) return sx_launch(heads_prepare_kernel<float>, grid, dim3(128), 0, stream, a);
  if (dt == SX_BF16) return sx_launch(heads_prepare_kernel<bf16>, grid, dim3(128), 0, stream, a);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// the attention
// ---------------------------------------------------------------------------------------
#define SC_THREADS 256
#define SC_KT 32                 // keys a tile: a lane a key where a warp works on one head

struct ScArgs {
  const void* q; const void* k_pages; const void* v_pages; void* out; float* part; float* part_ml;
  const int* positions; const int* seq_of_token; const int* block_table; int maxp;
  const int* tile_tok0; const int* tile_rows;
  int H, G, dim, vdim; float scale; int window;
  const float* talk; const float* head_bias; const float* dist_bias; int dist_n;
  int softmax; int n_chunks; int out_stride; const float* gate;
};

template <typename T> struct sc_io;
template <> struct sc_io<bf16> {
  static constexpr int KV = 8;        // elements of a 16-byte load
  static __device__ __forceinline__ void ld16(const bf16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
  static __device__ __forceinline__ void ld4(const bf16* p, float* f) {      // four elements
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 x = __bfloat1622float2(h[0]), y = __bfloat1622float2(h[1]);
    f[0] = x.x; f[1] = x.y; f[2] = y.x; f[3] = y.y;
  }
};
template <> struct sc_io<float> {
  static constexpr int KV = 4;
  static __device__ __forceinline__ void ld16(const float* p, float* f) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void ld4(const float* p, float* f) { ld16(p, f); }
};

// R: query heads of one item (they share a kv head); TQ: queries a block (consecutive rows of one sequence)
template <typename T, int R, int TQ>
__global__ void __launch_bounds__(SC_THREADS) attn_scored_kernel(const ScArgs a) {
  extern __shared__ __align__(16) unsigned char sc_smem[];
  pdl_wait();
  pdl_trigger();
  constexpr int KV = sc_io<T>::KV;
  const int H = a.H, G = a.G, dim = a.dim, vdim = a.vdim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = a.tile_tok0 ? a.tile_tok0[blockIdx.x] : blockIdx.x;
  const int rows = a.tile_tok0 ? min(TQ, a.tile_rows[blockIdx.x]) : 1;
  const int chunk = blockIdx.y;

  // shared memory: q [TQ][H][dim] as stored, S and P [TQ][H][32] float, talk [H][H], corr / m / l [TQ][H]
  const int qbytes = (TQ * H * dim * (int)sizeof(T) + 15) & ~15;
  T* qs = reinterpret_cast<T*>(sc_smem);
  float* S = reinterpret_cast<float*>(sc_smem + qbytes);
  float* P = S + TQ * H * SC_KT;
  float* talk = P + TQ * H * SC_KT;
  float* corr = talk + (a.talk ? H * H : 0);
  float* mrun = corr + TQ * H;
  float* lrun = mrun + TQ * H;
  __shared__ int pos_q[TQ];

  for (int i = tid; i < TQ * H * dim; i += SC_THREADS) {
    const int tq = i / (H * dim);
    qs[i] = tq < rows ? reinterpret_cast<const T*>(a.q)[(size_t)(tok0 + tq) * H * dim + (i - tq * H * dim)] : from_f32<T>(0.f);
  }
  if (a.talk) for (int i = tid; i < H * H; i += SC_THREADS) talk[i] = a.talk[i];
  for (int i = tid; i < TQ * H; i += SC_THREADS) { corr[i] = 1.f; mrun[i] = -INFINITY; lrun[i] = 0.f; }
  if (tid < TQ) pos_q[tid] = tid < rows ? a.positions[tok0 + tid] : -1;
  __syncthreads();

  const int first_pos = pos_q[0], last_pos = pos_q[rows - 1];
  const int lo = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;
  const int* bt = a.block_table + (size_t)a.seq_of_token[tok0] * a.maxp;
  const int tile_lo = lo >> 5, n_tiles = (last_pos >> 5) - tile_lo + 1;
  const int per = (n_tiles + a.n_chunks - 1) / a.n_chunks;
  const int tile_a = tile_lo + chunk * per, tile_b = min(tile_lo + n_tiles, tile_a + per);

  // what this thread accumulates: heads hg*R .. hg*R+R-1, value elements d0 .. d0+3
  const int nd = (vdim + 3) >> 2;
  const int item = blockIdx.z * SC_THREADS + tid;
  const bool own = item < (H / R) * nd;
  const int hg3 = own ? item / nd : 0, d0 = own ? (item - hg3 * nd) * 4 : 0;
  const int c3 = (hg3 * R) / (H / G);
  const bool vvec = (vdim & 3) == 0 && (((uintptr_t)a.v_pages) & 15) == 0;
  const bool kvec = dim % KV == 0 && (((uintptr_t)a.k_pages) & 15) == 0;
  float acc[TQ][R][4];
#pragma unroll
  for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[tq][r][0] = acc[tq][r][1] = acc[tq][r][2] = acc[tq][r][3] = 0.f;

  const T* kp = reinterpret_cast<const T*>(a.k_pages);
  const T* vp = reinterpret_cast<const T*>(a.v_pages);
  for (int tile = tile_a; tile < tile_b; ++tile) {
    const int j0 = tile << 5;
    const int page = bt[j0 >> 6];
    const int prow = j0 & 63;
    if (TQ == 1) {
      // a single token's step waits on memory: the tile's values are asked for now and come from L2 in part 3
      const int lines = (vdim * (int)sizeof(T) + 127) >> 7;
      for (int i = tid; i < G * SC_KT * lines; i += SC_THREADS) {
        const int ln = i % lines, j = (i / lines) % SC_KT, c = i / (lines * SC_KT);
        if (j0 + j <= last_pos && j0 + j >= lo)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(vp + (((size_t)page * G + c) * SX_PAGE + prow + j) * vdim + ln * (128 / sizeof(T))));
      }
    }
    // 1: raw scores of every head, a thread a (group of R heads, key)
    for (int it = tid; it < (H / R) * SC_KT; it += SC_THREADS) {
      const int hg = it >> 5, j = it & 31;
      const int c = (hg * R) / (H / G);
      float s[TQ][R];
#pragma unroll
      for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
        for (int r = 0; r < R; ++r) s[tq][r] = 0.f;
      if (j0 + j <= last_pos) {
        const T* kr = kp + (((size_t)page * G + c) * SX_PAGE + prow + j) * dim;
        if (kvec) {
#pragma unroll 8
          for (int d = 0; d < dim; d += KV) {            // (unrolled: several 16-byte loads of the key in flight)
            float kf[KV];
            sc_io<T>::ld16(kr + d, kf);
#pragma unroll
            for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
              for (int r = 0; r < R; ++r) {
                float qf[KV];
                sc_io<T>::ld16(qs + (size_t)(tq * H + hg * R + r) * dim + d, qf);
#pragma unroll
                for (int e = 0; e < KV; ++e) s[tq][r] = fmaf(qf[e], kf[e], s[tq][r]);
              }
          }
        } else {
          for (int d = 0; d < dim; ++d) {
            const float kf = to_f32(kr[d]);
#pragma unroll
            for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
              for (int r = 0; r < R; ++r) s[tq][r] = fmaf(to_f32(qs[(size_t)(tq * H + hg * R + r) * dim + d]), kf, s[tq][r]);
          }
        }
      }
#pragma unroll
      for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
        for (int r = 0; r < R; ++r) S[(tq * H + hg * R + r) * SC_KT + j] = s[tq][r] * a.scale;
    }
    __syncthreads();
    // 2: mixture over heads, biases, weights: a warp a (query, head), a lane a key
    for (int p = warp; p < TQ * H; p += SC_THREADS / 32) {
      const int tq = p / H, h = p - tq * H;
      const int pq = pos_q[tq], jk = j0 + lane;
      const bool vis = pq >= 0 && jk <= pq && (a.window == 0 || jk > pq - a.window);
      float s;
      if (a.talk) {
        s = 0.f;
        const float* tr = talk + h * H;
        const float* sr = S + tq * H * SC_KT + lane;
        for (int g = 0; g < H; ++g) s = fmaf(tr[g], sr[g * SC_KT], s);
      } else {
        s = S[p * SC_KT + lane];
      }
      if (a.head_bias) s += a.head_bias[h];
      if (a.dist_bias && vis) s += a.dist_bias[(size_t)h * a.dist_n + min(pq - jk, a.dist_n - 1)];
      float w;
      if (!a.softmax) {
        w = vis ? sigmoid_acc(s) : 0.f;
      } else {
        s = vis ? s : -INFINITY;
        const float m_old = mrun[p];
        const float m_new = fmaxf(m_old, warp_max(s));
        w = (m_new == -INFINITY) ? 0.f : expf(s - m_new);
        const float cr = (m_old == -INFINITY) ? 1.f : expf(m_old - m_new);
        const float ws = warp_sum(w);
        if (lane == 0) { corr[p] = cr; mrun[p] = m_new; lrun[p] = lrun[p] * cr + ws; }
      }
      P[p * SC_KT + lane] = w;
    }
    __syncthreads();
    // 3: weighted sums of the values
    if (own) {
      if (a.softmax) {
#pragma unroll
        for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float cr = corr[tq * H + hg3 * R + r];
            acc[tq][r][0] *= cr; acc[tq][r][1] *= cr; acc[tq][r][2] *= cr; acc[tq][r][3] *= cr;
          }
      }
      const int nj = min(SC_KT, last_pos - j0 + 1);
      const T* vr0 = vp + (((size_t)page * G + c3) * SX_PAGE + prow) * vdim + d0;
#pragma unroll 2
      for (int j = 0; j < nj; j += 4) {
        float vf[4][4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          if (j + jj < nj && j0 + j + jj >= lo) {            // keys before the window's edge may lie in memory nobody wrote
            if (vvec) {
              sc_io<T>::ld4(vr0 + (size_t)(j + jj) * vdim, vf[jj]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) vf[jj][e] = d0 + e < vdim ? to_f32(vr0[(size_t)(j + jj) * vdim + e]) : 0.f;
            }
          } else {
            vf[jj][0] = vf[jj][1] = vf[jj][2] = vf[jj][3] = 0.f;
          }
        }
#pragma unroll
        for (int tq = 0; tq < TQ; ++tq)
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float4 pw = *reinterpret_cast<const float4*>(P + (tq * H + hg3 * R + r) * SC_KT + j);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              acc[tq][r][e] = fmaf(pw.x, vf[0][e], fmaf(pw.y, vf[1][e], fmaf(pw.z, vf[2][e], fmaf(pw.w, vf[3][e], acc[tq][r][e]))));
          }
      }
    }
    __syncthreads();
  }

  if (!own) return;
  if (a.n_chunks == 1) {
#pragma unroll
    for (int tq = 0; tq < TQ; ++tq) {
      if (tq >= rows) continue;
      T* o = reinterpret_cast<T*>(a.out) + (size_t)(tok0 + tq) * a.out_stride;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int h = hg3 * R + r;
        float f = 1.f;
        if (a.softmax) { const float l = lrun[tq * H + h]; f = l > 0.f ? 1.f / l : 0.f; }
        if (a.gate) f *= a.gate[(size_t)(tok0 + tq) * H + h];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (d0 + e < vdim) o[(size_t)h * vdim + d0 + e] = from_f32<T>(acc[tq][r][e] * f);
      }
    }
    return;
  }
  // several chunks of the keys (TQ == 1): unnormalised sums, running maxima and sums of weights for the merge
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int h = hg3 * R + r;
    float* po = a.part + ((size_t)tok0 * a.n_chunks + chunk) * H * vdim + (size_t)h * vdim;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (d0 + e < vdim) po[d0 + e] = acc[0][r][e];
    if (a.softmax && d0 == 0) {
      float* ml = a.part_ml + (((size_t)tok0 * a.n_chunks + chunk) * H + h) * 2;
      ml[0] = mrun[h];
      ml[1] = lrun[h];
    }
  }
}

// the chunks of a token's keys added up in chunk order: a block a (token, head), a thread a value element
template <typename T>
__global__ void __launch_bounds__(128) attn_scored_merge_kernel(const float* __restrict__ part, const float* __restrict__ part_ml,
                                                                T* __restrict__ out, const float* __restrict__ gate, int H, int vdim,
                                                                int n_chunks, int softmax, int out_stride) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y;
  __shared__ float fac[64];
  __shared__ float red[33];
  float inv_l = 1.f;
  if (softmax) {
    // the parts' factors exp(m_c - m) once, by the first threads (n_chunks <= 64 <= blockDim.x is not required)
    float m = -INFINITY;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) m = fmaxf(m, part_ml[(((size_t)t * n_chunks + c) * H + h) * 2]);
    m = block_max(m, red);
    float l = 0.f;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
      const float* ml = part_ml + (((size_t)t * n_chunks + c) * H + h) * 2;
      const float f = ml[0] == -INFINITY ? 0.f : expf(ml[0] - m);
      fac[c] = f;
      l = fmaf(f, ml[1], l);
    }
    l = block_sum(l, red);
    inv_l = l > 0.f ? 1.f / l : 0.f;
  }
  const float g = gate ? gate[(size_t)t * H + h] : 1.f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    const float* p = part + (size_t)t * n_chunks * H * vdim + h * vdim + d;
    float o = 0.f;
#pragma unroll 16
    for (int c = 0; c < n_chunks; ++c) o = fmaf(softmax ? fac[c] : 1.f, p[(size_t)c * H * vdim], o);
    out[(size_t)t * out_stride + h * vdim + d] = from_f32<T>(o * inv_l * g);
  }
}

template <typename T, int R, int TQ>
static int scored_launch(const ScArgs& a, int n_tiles, cudaStream_t stream) {
  const int H = a.H;
  size_t smem = ((size_t)TQ * H * a.dim * sizeof(T) + 15) & ~(size_t)15;
  smem += (size_t)(2 * TQ * H * SC_KT + (a.talk ? H * H : 0) + 3 * TQ * H) * sizeof(float);
  if (smem > 200 * 1024) return SX_ERR_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_scored_kernel<T, R, TQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int nd = (a.vdim + 3) / 4;
  const int items = (H / R) * nd;
  dim3 grid(n_tiles, a.n_chunks, (items + SC_THREADS - 1) / SC_THREADS);
  return sx_launch(attn_scored_kernel<T, R, TQ>, grid, dim3(SC_THREADS), smem, stream, a);
}

template <typename T, int TQ>
static int scored_pick(const ScArgs& a, int n_tiles, cudaStream_t stream) {
  const int per = a.H / a.G;
  if (per % 4 == 0) return scored_launch<T, 4, TQ>(a, n_tiles, stream);
  if (per % 2 == 0) return scored_launch<T, 2, TQ>(a, n_tiles, stream);
  return scored_launch<T, 1, TQ>(a, n_tiles, stream);
}

// tile_tok0 / tile_rows null: a tile is one token (n_tiles = tokens) and the keys may be cut into n_chunks parts
// (part: float32 [tokens, n_chunks, H, vdim]; part_ml: float32 [tokens, n_chunks, H, 2], softmax only).
// Otherwise a tile is up to `tq` (1 or 4) consecutive rows of one sequence and n_chunks must be 1.
extern "C" int sx_attn_scored(const void* q, const void* k_pages, const void* v_pages, void* out, float* part, float* part_ml,
                              const int* positions, const int* seq_of_token, const int* block_table, int maxp,
                              const int* tile_tok0, const int* tile_rows, int n_tiles, int tq, int n_tokens, int H, int G, int dim,
                              int vdim, float scale, int window, const float* talk, const float* head_bias,
                              const float* dist_bias, int dist_n, int softmax, int n_chunks, int out_stride, const float* gate,
                              int dt, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || out_stride < H * vdim || n_chunks < 1 || H > 256) return SX_ERR_SIZE;
  if ((tq != 1 && tq != 4) || (tile_tok0 == nullptr && tq != 1) || (n_chunks > 1 && (tq != 1 || tile_tok0 || !part)))
    return SX_ERR_SIZE;
  if (n_chunks > 1 && softmax && !part_ml) return SX_ERR_SIZE;
  if (n_chunks > 64) return SX_ERR_SIZE;                       // the merge keeps a factor per part in shared memory
  if (dist_bias && dist_n <= 0) return SX_ERR_SIZE;
  ScArgs a;
  a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.out = out; a.part = part; a.part_ml = part_ml;
  a.positions = positions; a.seq_of_token = seq_of_token; a.block_table = block_table; a.maxp = maxp;
  a.tile_tok0 = tile_tok0; a.tile_rows = tile_rows; a.H = H; a.G = G; a.dim = dim; a.vdim = vdim; a.scale = scale;
  a.window = window; a.talk = talk; a.head_bias = head_bias; a.dist_bias = dist_bias; a.dist_n = dist_n;
  a.softmax = softmax; a.n_chunks = n_chunks; a.out_stride = out_stride; a.gate = n_chunks == 1 ? gate : nullptr;
  int rc;
  if (dt == SX_F32) rc = tq == 4 ? scored_pick<float, 4>(a, n_tiles, stream) : scored_pick<float, 1>(a, n_tiles, stream);
  else if (dt == SX_BF16) rc = tq == 4 ? scored_pick<bf16, 4>(a, n_tiles, stream) : scored_pick<bf16, 1>(a, n_tiles, stream);
  else return SX_ERR_DTYPE;
  if (rc != 0 || n_chunks == 1) return rc;
  const int mt = vdim <= 32 ? 32 : (vdim <= 64 ? 64 : 128);
  if (dt == SX_F32)
    return sx_launch(attn_scored_merge_kernel<float>, dim3(n_tokens, H), dim3(mt), 0, stream, (const float*)part,
                     (const float*)part_ml, (float*)out, gate, H, vdim, n_chunks, softmax, out_stride);
  return sx_launch(attn_scored_merge_kernel<bf16>, dim3(n_tokens, H), dim3(mt), 0, stream, (const float*)part,
                   (const float*)part_ml, (bf16*)out, gate, H, vdim, n_chunks, softmax, out_stride);
}

// =======================================================================================
// Prompt portions with sigmoid weights on the tensor cores (bfloat16 cache, mma.sync m16n8k16).
//
// A block takes up to 8 consecutive rows of one sequence and ALL heads, and walks the visible keys 16 at a time:
//   1  raw scores, keys as the rows of the product:  S^T_g [16 keys x 8 queries] = K_kv(g) [16 x dim] Q_g^T, into
//      shared memory as float32 times scale (warp w: heads w * HPW ..);
//   2  the mixture over heads in FFMA, a thread a (key, query) pair and half of the heads; bias, mask, sigmoid; the
//      weights go to shared memory as bfloat16 [head][query][key];
//   3  O^T_h [vdim x 8 queries] += V_kv(h)^T [vdim x 16 keys] P_h^T  (warp w: the same heads; the sums stay in registers,
//      HPW * vdim / 4 of them a thread, which is what limits a block to 8 rows).
// The next keys are fetched while the scores are mixed, the values while the raw scores are formed.
// H = 8 * HPW heads exactly; DIM and VD are 32, 64 or 128.
// =======================================================================================
#include "attn_tile.cuh"

#define TK_THREADS 256
#define TK_KT 16
#define TK_TQ 8

template <int HPW, int DIM, int VD> struct TkLayout {
  static constexpr int H = 8 * HPW;
  static constexpr int QROW = DIM * 2 + 16, VROW = VD * 2 + 16, PROW = TK_KT * 2 + 16;
  static constexpr int Q_BYTES = H * TK_TQ * QROW;
  static constexpr int S_BYTES = H * TK_KT * TK_TQ * 4;
  static constexpr int P_BYTES = H * TK_TQ * PROW;
  static constexpr int T_BYTES = H * H * 4;
  static size_t bytes(int G) { return (size_t)Q_BYTES + S_BYTES + P_BYTES + T_BYTES + (size_t)G * TK_KT * (QROW + VROW); }
};

struct TkArgs {
  const bf16* q; const bf16* k_pages; const bf16* v_pages; bf16* out;
  const int* positions; const int* seq_of_token; const int* block_table; int maxp;
  const int* tile_tok0; const int* tile_rows;
  int G; float scale; int window;
  const float* talk; const float* head_bias; const float* gate; int out_stride;
  float* part; int n_chunks;      // n_chunks > 1: the keys in that many parts over blockIdx.y, sums to part [tokens, n_chunks, H, vdim]
};

// rows j0 .. j0+15 of every kv head's page -> dst [G][16][ROWB]; rows outside [lo, hi] are zero-filled
template <int ELEMS, int ROWB>
__device__ __forceinline__ void tk_load(unsigned char* dst, const bf16* pages, int page, int G, int j0, int lo, int hi) {
  constexpr int CH = ELEMS / 8;
  const int prow = j0 & 63;
  for (int i = threadIdx.x; i < G * TK_KT * CH; i += TK_THREADS) {
    const int ch = i % CH, r = (i / CH) % TK_KT, c = i / (CH * TK_KT);
    const bool ok = j0 + r >= lo && j0 + r <= hi;
    const bf16* src = pages + (((size_t)page * G + c) * SX_PAGE + prow + (ok ? r : 0)) * ELEMS + ch * 8;
    cp_async16(smem_addr(dst + ((size_t)c * TK_KT + r) * ROWB + ch * 16), src, ok);
  }
}

template <int HPW, int DIM, int VD>
__global__ void __launch_bounds__(TK_THREADS, 1) attn_talk_prefill_kernel(const TkArgs a) {
  using L = TkLayout<HPW, DIM, VD>;
  constexpr int H = L::H;
  extern __shared__ __align__(16) unsigned char tk_smem[];
  __shared__ int pos_q[TK_TQ];
  pdl_wait();
  pdl_trigger();
  unsigned char* Qs = tk_smem;
  float* S = reinterpret_cast<float*>(Qs + L::Q_BYTES);
  unsigned char* Ps = reinterpret_cast<unsigned char*>(S) + L::S_BYTES;
  float* talk = reinterpret_cast<float*>(Ps + L::P_BYTES);
  unsigned char* Ks = reinterpret_cast<unsigned char*>(talk) + L::T_BYTES;
  const int G = a.G, per = H / G;
  unsigned char* Vs = Ks + (size_t)G * TK_KT * L::QROW;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int tile = gridDim.x - 1 - blockIdx.x;               // late rows see the most keys: first
  const int tok0 = a.tile_tok0 ? a.tile_tok0[tile] : tile;    // no tiles given: a block a token
  const int rows = a.tile_tok0 ? min(TK_TQ, a.tile_rows[tile]) : 1;
  if (tid < TK_TQ) pos_q[tid] = tid < rows ? a.positions[tok0 + tid] : -1;
  const int first_pos = a.positions[tok0], last_pos = first_pos + rows - 1;
  const int lo = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;
  const int* bt = a.block_table + (size_t)a.seq_of_token[tok0] * a.maxp;
  int j_begin = lo & ~(TK_KT - 1), j_end = last_pos + 1;       // this block's keys: j_begin <= j < j_end, 16 a turn
  if (a.n_chunks > 1) {
    const int turns = ((last_pos - j_begin) >> 4) + 1, per_chunk = (turns + a.n_chunks - 1) / a.n_chunks;
    j_end = min(j_end, j_begin + ((int)blockIdx.y + 1) * per_chunk * TK_KT);
    j_begin += (int)blockIdx.y * per_chunk * TK_KT;
    if (j_begin >= j_end) {                                    // a part without keys adds nothing
      for (int i = tid; i < rows * H * VD; i += TK_THREADS)
        a.part[((size_t)(tok0 + i / (H * VD)) * a.n_chunks + blockIdx.y) * H * VD + i % (H * VD)] = 0.f;
      return;
    }
  }

  // queries: [head][row][dim], rows beyond the tile zero
  for (int i = tid; i < H * TK_TQ * (DIM / 8); i += TK_THREADS) {
    const int ch = i % (DIM / 8), r = (i / (DIM / 8)) % TK_TQ, h = i / (DIM / 8 * TK_TQ);
    const bool ok = r < rows;
    cp_async16(smem_addr(Qs + ((size_t)h * TK_TQ + r) * L::QROW + ch * 16),
               a.q + ((size_t)(tok0 + (ok ? r : 0)) * H + h) * DIM + ch * 8, ok);
  }
  tk_load<DIM, L::QROW>(Ks, a.k_pages, bt[j_begin >> 6], G, j_begin, lo, last_pos);
  cp_async_commit();
  for (int i = tid; i < H * H; i += TK_THREADS) talk[i] = a.talk ? a.talk[i] : ((i / H == i % H) ? 1.f : 0.f);

  float o[HPW][VD / 16][4];
#pragma unroll
  for (int r = 0; r < HPW; ++r)
#pragma unroll
    for (int n = 0; n < VD / 16; ++n) o[r][n][0] = o[r][n][1] = o[r][n][2] = o[r][n][3] = 0.f;

  for (int j0 = j_begin; j0 < j_end; j0 += TK_KT) {
    tk_load<VD, L::VROW>(Vs, a.v_pages, bt[j0 >> 6], G, j0, lo, last_pos);
    cp_async_commit();
    cp_async_wait<1>();                                       // the keys (and, the first time, the queries)
    __syncthreads();
    // 1: raw scores
#pragma unroll
    for (int r = 0; r < HPW; ++r) {
      const int h = warp * HPW + r, c = h / per;
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t ka = smem_addr(Ks + ((size_t)c * TK_KT + (lane & 7) + ((lane >> 3) & 1) * 8) * L::QROW + (lane >> 4) * 16);
      const uint32_t qa = smem_addr(Qs + ((size_t)h * TK_TQ + (lane & 7)) * L::QROW + (lane >> 3) * 16);
#pragma unroll
      for (int d = 0; d < DIM / 32; ++d) {
        uint32_t b0, b1, b2, b3, a0[4], a1[4];
        ldsm_x4(b0, b1, b2, b3, qa + d * 64);
        ldsm_x4(a0[0], a0[1], a0[2], a0[3], ka + d * 64);
        ldsm_x4(a1[0], a1[1], a1[2], a1[3], ka + d * 64 + 32);
        mma16816(s, a0, b0, b1);
        mma16816(s, a1, b2, b3);
      }
      float* sh = S + h * (TK_KT * TK_TQ);
      *reinterpret_cast<float2*>(sh + g * TK_TQ + 2 * t) = make_float2(s[0] * a.scale, s[1] * a.scale);
      *reinterpret_cast<float2*>(sh + (g + 8) * TK_TQ + 2 * t) = make_float2(s[2] * a.scale, s[3] * a.scale);
    }
    __syncthreads();
    if (j0 + TK_KT < j_end) tk_load<DIM, L::QROW>(Ks, a.k_pages, bt[(j0 + TK_KT) >> 6], G, j0 + TK_KT, lo, last_pos);
    cp_async_commit();
    // 2: mixture over heads, bias, mask, sigmoid
    {
      const int pair = tid & (TK_KT * TK_TQ - 1), half = tid >> 7;
      const int key = pair >> 3, qi = pair & 7;
      const int pq = pos_q[qi], jk = j0 + key;
      const bool vis = pq >= 0 && jk <= pq && (a.window == 0 || jk > pq - a.window);
      float raw[H];
#pragma unroll
      for (int gg = 0; gg < H; ++gg) raw[gg] = S[gg * (TK_KT * TK_TQ) + pair];
      // four heads at a time: four independent chains of FFMA, their rows of the matrix loaded together
      constexpr int HB = (H / 2) % 4 == 0 ? 4 : (H / 2) % 2 == 0 ? 2 : 1;
#pragma unroll
      for (int hh = 0; hh < H / 2; hh += HB) {
        const int h0 = half * (H / 2) + hh;
        float acc[HB];
#pragma unroll
        for (int u = 0; u < HB; ++u) acc[u] = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < H / 4; ++g4) {
          float4 w4[HB];
#pragma unroll
          for (int u = 0; u < HB; ++u) w4[u] = reinterpret_cast<const float4*>(talk + (h0 + u) * H)[g4];
#pragma unroll
          for (int u = 0; u < HB; ++u) acc[u] = fmaf(w4[u].x, raw[4 * g4], acc[u]);
#pragma unroll
          for (int u = 0; u < HB; ++u) acc[u] = fmaf(w4[u].y, raw[4 * g4 + 1], acc[u]);
#pragma unroll
          for (int u = 0; u < HB; ++u) acc[u] = fmaf(w4[u].z, raw[4 * g4 + 2], acc[u]);
#pragma unroll
          for (int u = 0; u < HB; ++u) acc[u] = fmaf(w4[u].w, raw[4 * g4 + 3], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < HB; ++u) {
          const int h = h0 + u;
          if (a.head_bias) acc[u] += a.head_bias[h];
          // the weight becomes a bfloat16 operand: the fast exponential's and division's few units in the last place of
          // 32 bits are far below its rounding
          const float w = vis ? __fdividef(1.f, 1.f + __expf(-acc[u])) : 0.f;
          *reinterpret_cast<bf16*>(Ps + ((size_t)h * TK_TQ + qi) * L::PROW + key * 2) = __float2bfloat16_rn(w);
        }
      }
    }
    cp_async_wait<1>();                                       // the values
    __syncthreads();
    // 3: weighted sums of the values
    {
      int c_have = -1;
      uint32_t va[VD / 16][4];
      const int lm = lane >> 3;
#pragma unroll
      for (int r = 0; r < HPW; ++r) {
        const int h = warp * HPW + r, c = h / per;
        if (c != c_have) {
          c_have = c;
          const uint32_t vaddr = smem_addr(Vs + ((size_t)c * TK_KT + (lane & 7) + (lm >> 1) * 8) * L::VROW + (lm & 1) * 16);
#pragma unroll
          for (int n = 0; n < VD / 16; ++n) ldsm_x4_trans(va[n][0], va[n][1], va[n][2], va[n][3], vaddr + n * 32);
        }
        const unsigned char* pr = Ps + ((size_t)h * TK_TQ + g) * L::PROW + 4 * t;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(pr), b1 = *reinterpret_cast<const uint32_t*>(pr + 16);
#pragma unroll
        for (int n = 0; n < VD / 16; ++n) mma16816(o[r][n], va[n], b0, b1);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // o[r][n]: value elements n*16 + g (+8) of queries 2t, 2t+1
#pragma unroll
  for (int r = 0; r < HPW; ++r) {
    const int h = warp * HPW + r;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qi = 2 * t + e;
      if (qi >= rows) continue;
      if (a.n_chunks > 1) {                                   // (the gate is applied where the parts are added)
        float* prow = a.part + ((size_t)(tok0 + qi) * a.n_chunks + blockIdx.y) * H * VD + (size_t)h * VD;
#pragma unroll
        for (int n = 0; n < VD / 16; ++n) {
          prow[n * 16 + g] = o[r][n][e];
          prow[n * 16 + g + 8] = o[r][n][2 + e];
        }
        continue;
      }
      const float f = a.gate ? a.gate[(size_t)(tok0 + qi) * H + h] : 1.f;
      bf16* orow = a.out + (size_t)(tok0 + qi) * a.out_stride + (size_t)h * VD;
#pragma unroll
      for (int n = 0; n < VD / 16; ++n) {
        orow[n * 16 + g] = __float2bfloat16_rn(o[r][n][e] * f);
        orow[n * 16 + g + 8] = __float2bfloat16_rn(o[r][n][2 + e] * f);
      }
    }
  }
}

template <int HPW, int DIM, int VD>
static int talk_launch(const TkArgs& a, int n_tiles, cudaStream_t stream) {
  const size_t smem = TkLayout<HPW, DIM, VD>::bytes(a.G);
  if (smem > 220 * 1024) return SX_ERR_SIZE;
  cudaError_t e = cudaFuncSetAttribute(attn_talk_prefill_kernel<HPW, DIM, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return sx_launch(attn_talk_prefill_kernel<HPW, DIM, VD>, dim3(n_tiles, a.n_chunks), dim3(TK_THREADS), smem, stream, a);
}

template <int HPW, int DIM>
static int talk_pick_v(const TkArgs& a, int n_tiles, int vdim, cudaStream_t stream) {
  if (vdim == 128) return talk_launch<HPW, DIM, 128>(a, n_tiles, stream);
  if (vdim == 64) return talk_launch<HPW, DIM, 64>(a, n_tiles, stream);
  if (vdim == 32) return talk_launch<HPW, DIM, 32>(a, n_tiles, stream);
  return SX_ERR_SIZE;
}
template <int HPW>
static int talk_pick(const TkArgs& a, int n_tiles, int dim, int vdim, cudaStream_t stream) {
  if (dim == 128) return talk_pick_v<HPW, 128>(a, n_tiles, vdim, stream);
  if (dim == 64) return talk_pick_v<HPW, 64>(a, n_tiles, vdim, stream);
  if (dim == 32) return talk_pick_v<HPW, 32>(a, n_tiles, vdim, stream);
  return SX_ERR_SIZE;
}

// bytes of shared memory a block of the tensor-core prompt kernel needs, or -1 where it does not apply
extern "C" int sx_attn_talk_prefill_smem(int H, int G, int dim, int vdim) {
  if ((H != 8 && H != 16 && H != 32) || G <= 0 || H % G || (dim != 32 && dim != 64 && dim != 128) ||
      (vdim != 32 && vdim != 64 && vdim != 128))
    return -1;
  const size_t row = (size_t)dim * 2 + 16, vrow = (size_t)vdim * 2 + 16;
  return (int)((size_t)H * TK_TQ * row + (size_t)H * TK_KT * TK_TQ * 4 + (size_t)H * TK_TQ * (TK_KT * 2 + 16) +
                     (size_t)H * H * 4 + (size_t)G * TK_KT * (row + vrow));
}

// tiles: up to 8 consecutive rows of one sequence each; tile_tok0 null: a tile a token (n_tiles tokens), and then the
// keys may be cut into n_chunks <= 64 parts (part: float32 [tokens, n_chunks, H, vdim]) that a second kernel adds up.
// Sigmoid weights only; talk, head_bias and gate may be null.
extern "C" int sx_attn_talk_prefill(const void* q, const void* k_pages, const void* v_pages, void* out, const int* positions,
                                    const int* seq_of_token, const int* block_table, int maxp, const int* tile_tok0,
                                    const int* tile_rows, int n_tiles, int H, int G, int dim, int vdim, float scale, int window,
                                    const float* talk, const float* head_bias, const float* gate, int out_stride,
                                    float* part, int n_chunks, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (sx_attn_talk_prefill_smem(H, G, dim, vdim) < 0 || out_stride < H * vdim || (tile_tok0 == nullptr) != (tile_rows == nullptr))
    return SX_ERR_SIZE;
  if (n_chunks < 1 || n_chunks > 64 || (n_chunks > 1 && (tile_tok0 || !part))) return SX_ERR_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return SX_ERR_ALIGN;
  TkArgs a;
  a.q = (const bf16*)q; a.k_pages = (const bf16*)k_pages; a.v_pages = (const bf16*)v_pages; a.out = (bf16*)out;
  a.positions = positions; a.seq_of_token = seq_of_token; a.block_table = block_table; a.maxp = maxp;
  a.tile_tok0 = tile_tok0; a.tile_rows = tile_rows; a.G = G; a.scale = scale; a.window = window; a.talk = talk;
  a.head_bias = head_bias; a.gate = gate; a.out_stride = out_stride; a.part = part; a.n_chunks = n_chunks;
  const int rc = H == 32 ? talk_pick<4>(a, n_tiles, dim, vdim, stream)
               : H == 16 ? talk_pick<2>(a, n_tiles, dim, vdim, stream) : talk_pick<1>(a, n_tiles, dim, vdim, stream);
  if (rc != 0 || n_chunks == 1) return rc;
  const int mt = vdim <= 32 ? 32 : (vdim <= 64 ? 64 : 128);
  return sx_launch(attn_scored_merge_kernel<bf16>, dim3(n_tiles, H), dim3(mt), 0, stream, (const float*)part, (const float*)nullptr,
                   (bf16*)out, gate, H, vdim, n_chunks, 0, out_stride);
}
