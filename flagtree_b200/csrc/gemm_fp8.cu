// Block-scaled FP8 (e4m3) GEMM for sm_100a: C[M,N] = sum_kb (A[:,kb] . B[kb,:]) * a_scale[:,kb] (x) b_scale[kb,:/128]
// with A [M,K] e4m3 and 1x128 fp32 scales, B [K,N] e4m3 and 128x128 fp32 scales, bf16 output.
//
// The tensor cores' own block scaling takes 32-element ue8m0/ue4m3 scales, not fp32 per 128, so every
// 128-deep K block is multiplied on its own (4 tcgen05.mma kind::f8f6f4 of K = 32 into a fresh TMEM
// accumulator) and four "promotion" warps fold it into fp32 registers with its two scales while the
// next block is being multiplied (two TMEM accumulators of 128 columns).
// Tile 128 x 128, K step 128; A stage [128 rows x 128 B] K-major; B stage either [128 k-rows x 128 B]
// (128 columns; B given as [K, N] row-major, the MN-major operand) or [128 columns x 128 B] (B given as the
// transpose [N, K] row-major, as a linear layer keeps its weight: the K-major operand, same speed, same bits);
// 6 stages of 32 KB filled by TMA.
// Measured and not kept (cfg5 shapes, 908 / 1080 / 1090 TFLOP/s with this kernel; the tensor pipe is 32 % busy, L2
// 37 %): eight promotion warps with packed two-wide adds and the scales fetched a block ahead (-4 %), CTA pairs
// on 256 x 256 tiles (-20 %), four accumulators in flight instead of two (no change).
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 promotion/epilogue.
#include <cstring>

#include "sm100.cuh"
#include "tmap.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace gemm8 {

constexpr int BM = 128, BN = 128, BK = 128, STAGES = 6;
constexpr int A_BYTES = BM * BK;          // 16384
constexpr int B_BYTES = BK * BN;          // 16384
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;

struct Params {
  int m, n, k, n_blocks, n_tiles, kb_total;
  const float* a_scale;   // [m, kb_total]
  const float* b_scale;   // [kb_total, n / 128]
  long long lda_s, ldb_s;
  __nv_bfloat16* c;
  long long ldc;
  int* status;
};

struct Bars {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long blk_full[2];
  unsigned long long blk_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <bool B_KMAJOR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  Bars* bars = reinterpret_cast<Bars*>(sm + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    bars->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->blk_full[a]), 1);
      mbar_init(smem_u32(&bars->blk_empty[a]), 4);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (bars->abort_flag) return;
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 256);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
        const int m_blk = t / p.n_blocks, n_blk = t - m_blk * p.n_blocks;
        for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) & 1u) ^ 1u, abort_flag);
          const uint32_t full = smem_u32(&bars->full[s]);
          mbar_arrive_expect_tx(full, STAGE_BYTES);
          const uint32_t a_dst = base + s * STAGE_BYTES;
          tma_load_2d(a_dst, &tm_a, full, kb * BK, m_blk * BM);
          if constexpr (B_KMAJOR) tma_load_2d(a_dst + A_BYTES, &tm_b, full, kb * BK, n_blk * BN);
          else tma_load_2d(a_dst + A_BYTES, &tm_b, full, n_blk * BN, kb * BK);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t kIdesc = umma_idesc(kFmtE4M3, BM, BN, 0, B_KMAJOR ? 0 : 1);
      uint32_t it = 0;   // K blocks issued so far = accumulator uses
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
        for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t acc = it & 1u;
          mbar_wait(smem_u32(&bars->blk_empty[acc]), ((it >> 1) & 1u) ^ 1u, abort_flag);
          mbar_wait(smem_u32(&bars->full[s]), (it / STAGES) & 1u, abort_flag);
          tc_fence_after();
          const uint32_t a_s = base + s * STAGE_BYTES;
          const uint32_t b_s = a_s + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            const uint64_t ad = smem_desc_sw128(a_s + k * 32, 16, 1024);          // K-major: 32 B per K step
            const uint64_t bd = B_KMAJOR ? smem_desc_sw128(b_s + k * 32, 16, 1024)            // K-major: 32 B per K step
                                         : smem_desc_sw128(b_s + k * 4096, B_BYTES, 1024);   // MN-major: 32 k-rows per step
            umma_f8_ss(tmem + acc * BN, ad, bd, kIdesc, k != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars->empty[s]));
          umma_commit(smem_u32(&bars->blk_full[acc]));
        }
      }
    }
  } else {
    const int lg = warp & 3;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
      const int m_blk = t / p.n_blocks, n_blk = t - m_blk * p.n_blocks;
      const int row = m_blk * BM + lg * 32 + lane;
      const bool row_ok = row < p.m;
      float accf[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) accf[j] = 0.0f;
      const float* as_row = p.a_scale + static_cast<long long>(row_ok ? row : 0) * p.lda_s;
      for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
        const uint32_t acc = it & 1u;
        const float sc = as_row[kb] * p.b_scale[static_cast<long long>(kb) * p.ldb_s + n_blk];
        mbar_wait(smem_u32(&bars->blk_full[acc]), (it >> 1) & 1u, abort_flag);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c0), v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) accf[c0 + j] = fmaf(__uint_as_float(v[j]), sc, accf[c0 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->blk_empty[acc]));
      }
      if (row_ok) {
        __nv_bfloat16* orow = p.c + static_cast<long long>(row) * p.ldc + n_blk * BN;
#pragma unroll
        for (int j = 0; j < BN; j += 8) {
          if (n_blk * BN + j < p.n) {
            uint4 o;
            o.x = pack_bf16x2(accf[j], accf[j + 1]);
            o.y = pack_bf16x2(accf[j + 2], accf[j + 3]);
            o.z = pack_bf16x2(accf[j + 4], accf[j + 5]);
            o.w = pack_bf16x2(accf[j + 6], accf[j + 7]);
            *reinterpret_cast<uint4*>(orow + j) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (tid == 0 && p.status != nullptr && bars->abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
}

}  // namespace gemm8
}  // namespace ftb

using namespace ftb;

extern "C" FTB_API int ftb_gemm_fp8_blockscaled(const ftb_gemm_fp8_args* g, void* stream) {
  if (!g || !g->a || !g->b || !g->c || !g->a_scale || !g->b_scale) { set_last_error("ftb_gemm_fp8_blockscaled: null pointer"); return FTB_ERR_INVALID; }
  if (g->m <= 0 || g->n <= 0 || g->k <= 0 || (g->k % 128) || (g->n % 128)) {
    set_last_error("ftb_gemm_fp8_blockscaled: need k and n multiples of 128 (scale blocks), got m=%d n=%d k=%d", g->m, g->n, g->k);
    return FTB_ERR_INVALID;
  }
  if ((g->lda % 16) || (g->ldb % 16) || (g->ldc % 8) || (reinterpret_cast<uintptr_t>(g->a) & 15) ||
      (reinterpret_cast<uintptr_t>(g->b) & 15) || (reinterpret_cast<uintptr_t>(g->c) & 15)) {
    set_last_error("ftb_gemm_fp8_blockscaled: pointers must be 16-byte aligned, lda/ldb multiples of 16, ldc of 8");
    return FTB_ERR_INVALID;
  }
  CUtensorMap tm_a, tm_b;
  const bool bkm = g->b_kmajor != 0;
  if (!make_tmap_2d(&tm_a, g->a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g->m, g->k, g->lda, gemm8::BM, 128) ||
      !(bkm ? make_tmap_2d(&tm_b, g->b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g->n, g->k, g->ldb, gemm8::BN, 128)
            : make_tmap_2d(&tm_b, g->b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g->k, g->n, g->ldb, gemm8::BK, 128))) {
    set_last_error("ftb_gemm_fp8_blockscaled: cuTensorMapEncodeTiled failed");
    return FTB_ERR_CUDA;
  }
  gemm8::Params p;
  memset(&p, 0, sizeof(p));
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.n_blocks = g->n / gemm8::BN;
  p.n_tiles = ((g->m + gemm8::BM - 1) / gemm8::BM) * p.n_blocks;
  p.kb_total = g->k / gemm8::BK;
  p.a_scale = g->a_scale; p.b_scale = g->b_scale;
  p.lda_s = g->a_scale_ld; p.ldb_s = g->b_scale_ld;
  p.c = reinterpret_cast<__nv_bfloat16*>(g->c);
  p.ldc = g->ldc;
  p.status = g->status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  auto kern = bkm ? gemm8::gemm_fp8_kernel<true> : gemm8::gemm_fp8_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm_fp8)");
  const int grid = p.n_tiles < sms ? p.n_tiles : sms;
  kern<<<grid, gemm8::THREADS, gemm8::SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(tm_a, tm_b, p);
  return check_cuda(cudaGetLastError(), "gemm_fp8 launch");
}
