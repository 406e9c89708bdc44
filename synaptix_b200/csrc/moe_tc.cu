// The experts' grouped product on the 5th-generation tensor cores (sm_100a, bfloat16): the one-tile-a-block tcgen05
// product of this library with the rows of a tile taken from ONE expert's group.
//
// A [rows, K] holds the step's (token, choice) rows sorted by expert (offsets [E + 1] on the device); W [E, NW, K] the
// experts' matrices, seen by TMA as one [E * NW, K] matrix.  Block (x, y): y counts 128-row tiles expert by expert (a
// block finds its expert and first row from `offsets`; blocks beyond the last tile return), x counts column tiles.
// A tile's rows beyond its group's end belong to the next expert (or lie behind the matrix, where TMA fills zeros):
// they are computed and not stored.  TMA (128-byte swizzle) -> ring of stages -> tcgen05.mma 128 x 256 x 16 issued
// by one lane -> accumulator in tensor memory -> tcgen05.ld epilogue of four warps:
//   GATE_UP: the tile's 256 matrix rows are 128 gate rows and the 128 up rows of the same outputs; the epilogue
//            writes silu(gate) * up as bfloat16 [rows, N];
//   else:    the plain product as float32 [rows, N].
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word, and the block still frees its
// tensor memory.  K % 8 == 0 (TMA strides); a tail of K is zero-filled by TMA.
#include "tcgen05.cuh"

#define MT_BM 128
#define MT_BN 256
#define MT_BK 64
#define MT_A_BYTES (MT_BM * MT_BK * 2)
#define MT_B_BYTES (MT_BN * MT_BK * 2)
#define MT_STAGE_BYTES (MT_A_BYTES + MT_B_BYTES)
#define MT_STAGES 4
#define MT_THREADS 192

template <bool GATE_UP>
__global__ void __launch_bounds__(MT_THREADS, 1) moe_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_w,
                                                               void* __restrict__ out, const int* __restrict__ offsets,
                                                               int E, int N, int K, int* __restrict__ status, const GateAct act) {
  extern __shared__ unsigned char mt_smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(mt_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + MT_STAGES * MT_STAGE_BYTES);   // full[S], empty[S], accum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MT_STAGES + 1);
  int* which = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t full0 = tc_smem(bars), empty0 = tc_smem(bars + MT_STAGES), accum = tc_smem(bars + 2 * MT_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_wait();          // the offsets come from the kernel before
  pdl_trigger();
  if (threadIdx.x == 0) {
    int tile = blockIdx.y, e = 0, r0 = -1;
    for (; e < E; ++e) {
      const int n_e = offsets[e + 1] - offsets[e];
      const int t = (n_e + MT_BM - 1) / MT_BM;
      if (tile < t) { r0 = offsets[e] + tile * MT_BM; break; }
      tile -= t;
    }
    which[0] = e; which[1] = r0; which[2] = r0 >= 0 ? min(MT_BM, offsets[e + 1] - r0) : 0;
  }
  __syncthreads();
  const int e = which[0], m0 = which[1], nr = which[2];
  if (m0 < 0) return;                                   // the whole block: no barrier or tensor memory is held yet

  constexpr int tile_n = GATE_UP ? MT_BN / 2 : MT_BN;   // columns of the result per block
  const int NW = GATE_UP ? 2 * N : N;                   // rows of one expert's matrix
  const int n0 = blockIdx.x * tile_n;
  const int nkb = (K + MT_BK - 1) / MT_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MT_STAGES; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    tc_mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(tmem_slot)), "r"((uint32_t)MT_BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % MT_STAGES;
        if (!tc_mbar_wait(empty0 + 8 * s, ((kb / MT_STAGES) & 1) ^ 1)) { sx_set_status(status, 1); break; }
        tc_mbar_expect_tx(full0 + 8 * s, MT_STAGE_BYTES);
        const uint32_t a_dst = tc_smem(tiles + s * MT_STAGE_BYTES), b_dst = a_dst + MT_A_BYTES;
        const int kx = kb * MT_BK;
        tc_tma_load_2d(a_dst, &map_a, kx, m0, full0 + 8 * s);
        const int w0 = e * NW + n0;
        tc_tma_load_2d(b_dst, &map_w, kx, w0, full0 + 8 * s);                                          // gate rows (or the first 128)
        tc_tma_load_2d(b_dst + MT_B_BYTES / 2, &map_w, kx, w0 + (GATE_UP ? N : 128), full0 + 8 * s);   // up rows (or the next 128)
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instr_desc(MT_BM, MT_BN);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % MT_STAGES;
        if (!tc_mbar_wait(full0 + 8 * s, (kb / MT_STAGES) & 1)) { sx_set_status(status, 2); break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = tc_smem(tiles + s * MT_STAGE_BYTES), b_addr = a_addr + MT_A_BYTES;
#pragma unroll
        for (int k = 0; k < MT_BK / 16; ++k)
          tc_mma(tmem_base, tc_smem_desc(a_addr + k * 32), tc_smem_desc(b_addr + k * 32), idesc, (kb | k) != 0);
        tc_commit(empty0 + 8 * s);
      }
      tc_commit(accum);
    }
    __syncwarp();
  } else {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                   // row of the tile
    if (tc_mbar_wait(accum, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < tile_n; c0 += 32) {
        uint32_t v[32], u[32];
        tc_ld32(t_row + c0, v);
        if (GATE_UP) tc_ld32(t_row + MT_BN / 2 + c0, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (r >= nr || n0 + c0 >= N) continue;
        const int ncol = min(32, N - (n0 + c0));
        if (GATE_UP) {
          bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)(m0 + r) * N + n0 + c0;
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = __uint_as_float(v[i]);
            f[i] = gate_mul(g, __uint_as_float(u[i]), act);
          }
          if (ncol == 32 && (N % 8) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 p;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(f[8 * i], f[8 * i + 1]), t1 = __floats2bfloat162_rn(f[8 * i + 2], f[8 * i + 3]);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(f[8 * i + 4], f[8 * i + 5]), t3 = __floats2bfloat162_rn(f[8 * i + 6], f[8 * i + 7]);
              p.x = *reinterpret_cast<uint32_t*>(&t0); p.y = *reinterpret_cast<uint32_t*>(&t1);
              p.z = *reinterpret_cast<uint32_t*>(&t2); p.w = *reinterpret_cast<uint32_t*>(&t3);
              reinterpret_cast<uint4*>(dst)[i] = p;
            }
          } else {
            for (int i = 0; i < ncol; ++i) dst[i] = __float2bfloat16_rn(f[i]);
          }
        } else {
          float* dst = reinterpret_cast<float*>(out) + (size_t)(m0 + r) * N + n0 + c0;
          if (ncol == 32 && (N % 4) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                              __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
          } else {
            for (int i = 0; i < ncol; ++i) dst[i] = __uint_as_float(v[i]);
          }
        }
      }
    } else {
      if (lane == 0) sx_set_status(status, 3);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)MT_BN) : "memory");
  }
}

// rows of x gathered into sorted order: xs[p] = x[order[p] / top]
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ order, bf16* __restrict__ xs, int K, int top) {
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(order[p] / top) * K);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}

extern "C" int sx_moe_gather(const void* x, const int* order, void* xs, int rows, int K, int top, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K % 8 || (((uintptr_t)x | (uintptr_t)xs) % 16)) return SX_ERR_ALIGN;
  return sx_launch(moe_gather_kernel, dim3(rows), dim3(128), 0, stream, (const bf16*)x, order, (bf16*)xs, K, top);
}

static int* mt_status_word() {
  static int* w = nullptr;
  if (!w) w = sx_status_word_alloc();
  return w;
}

extern "C" int sx_moe_tc_status(int* host_value, int reset) {
  int* w = mt_status_word();
  if (!w) return SX_ERR_SIZE;
  *host_value = *(volatile int*)w;
  if (reset) *(volatile int*)w = 0;
  return 0;
}

extern "C" int sx_moe_tc(const void* A, const void* Wt, void* out, const int* offsets, int rows, int E, int N, int K,
                         int gate_up, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || N <= 0 || K <= 0 || K % 8) return SX_ERR_SIZE;
  if (((uintptr_t)A | (uintptr_t)Wt | (uintptr_t)out) % 16) return SX_ERR_ALIGN;
  int* status = mt_status_word();
  if (!status) return SX_ERR_SIZE;
  const int NW = gate_up ? 2 * N : N;
  CUtensorMap ma, mw;
  int rc = tc_make_map_rows(&ma, A, rows, K, MT_BM);
  if (rc) return rc;
  rc = tc_make_map_rows(&mw, Wt, (long long)E * NW, K, 128);
  if (rc) return rc;
  const int tiles = (rows + MT_BM - 1) / MT_BM + (E < rows ? E : rows);
  if (tiles > 65535) return SX_ERR_SIZE;
  const size_t smem = (size_t)MT_STAGES * MT_STAGE_BYTES + 1024 + (2 * MT_STAGES + 1) * 8 + 32;
  if (gate_up) {
    static bool set = false;
    if (!set) {
      cudaError_t err = cudaFuncSetAttribute(moe_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
      set = true;
    }
    return sx_launch(moe_tc_kernel<true>, dim3((N + MT_BN / 2 - 1) / (MT_BN / 2), tiles), dim3(MT_THREADS), smem, stream, ma, mw, out,
                     offsets, E, N, K, status, g_sx_gate);
  }
  static bool set2 = false;
  if (!set2) {
    cudaError_t err = cudaFuncSetAttribute(moe_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    set2 = true;
  }
  return sx_launch(moe_tc_kernel<false>, dim3((N + MT_BN - 1) / MT_BN, tiles), dim3(MT_THREADS), smem, stream, ma, mw, out, offsets, E,
                   N, K, status, g_sx_gate);
}
