// Persistent, warp-specialised tcgen05 GEMM for sm_100a: C[M,N] = A[M,K] . B[K,N], bf16 in, fp32
// accumulate in TMEM, bf16 out -- and the same kernel with a reduce-scatter epilogue: a finished tile
// whose rows belong to another rank is stored (TMA store from a staging box, never a multicast load)
// straight into that rank's receive slot in peer memory over NVLink and a per-(source, row block)
// counter is released; tiles of this rank's own rows are computed last and their epilogue adds the
// partials the other ranks have pushed (fixed order, fp32) before writing the bf16 shard.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM), warps 2-5 = epilogue.
// Tile 128 x 256, K step 64, 4 shared-memory stages of 48 KB, two 256-column TMEM accumulators so the
// epilogue of tile i overlaps the MMAs of tile i+1.
//   A stage: [128 rows x 128 B] K-major, 128B swizzle (one TMA box)
//   B stage: 4 blocks of [64 k-rows x 128 B] (64 N columns each), used as the MN-major operand.
#include <cstring>

#include "sm100.cuh"
#include "tmap.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;                 // 16384
constexpr int B_BLOCK_BYTES = BK * 128;              // 8192: 64 k-rows x 64 columns
constexpr int B_BYTES = (BN / 64) * B_BLOCK_BYTES;   // 32768
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;       // 49152
constexpr int STAGING_BYTES = 4 /*warps*/ * 2 /*buffers*/ * 4096;   // [32 rows x 128 B] boxes for TMA stores
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int THREADS = 192;
constexpr int MAX_TP = 8;

struct Params {
  int m, n, k;
  int n_blocks, m_blocks, n_tiles;
  // plain GEMM output
  __nv_bfloat16* c;
  long long ldc;
  // reduce-scatter output: rank `dst` receives rows [dst*shard_rows, (dst+1)*shard_rows)
  int tp, rank, shard_rows, blocks_per_shard;
  __nv_bfloat16* recv[MAX_TP];       // base of dst's receive buffer [tp][shard_rows][n] (peer-mapped)
  unsigned int* flags[MAX_TP];       // base of dst's flag array [tp][blocks_per_shard] then done[tp]
  unsigned int epoch;                // this call's sequence number (>= 1)
  unsigned int flag_target;          // value every (src, row block) counter reaches in this call
  __nv_bfloat16* out;                // this rank's shard [shard_rows, n]
  long long ldo;
  unsigned int* counter;             // CTA completion counter (device, zero between calls)
  int* status;
};

// One tensor map per destination rank: that rank's receive slot for THIS rank, [shard_rows, n] bf16.
struct OutMaps {
  CUtensorMap m[MAX_TP];
};

struct Bars {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(const Params& p, int t, int& m_blk, int& n_blk, int& dst) {
  if (p.tp <= 1) {
    m_blk = t / p.n_blocks;
    n_blk = t - m_blk * p.n_blocks;
    dst = 0;
    return;
  }
  const int per_shard = p.blocks_per_shard * p.n_blocks;
  const int ord = t / per_shard;                     // remote shards first, own shard last
  dst = (p.rank + 1 + ord) % p.tp;
  const int r = t - ord * per_shard;
  const int mb = r / p.n_blocks;
  n_blk = r - mb * p.n_blocks;
  m_blk = dst * p.blocks_per_shard + mb;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_pending4() { asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ OutMaps tm_out, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  Bars* bars = reinterpret_cast<Bars*>(sm + STAGES * STAGE_BYTES + STAGING_BYTES);
  const uint32_t staging = base + STAGES * STAGE_BYTES;
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int kb_total = (p.k + BK - 1) / BK;

  if (tid == 0) {
    bars->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->acc_full[a]), 1);
      mbar_init(smem_u32(&bars->acc_empty[a]), 4);   // one arrival per epilogue warp
    }
    fence_mbar_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  __syncthreads();
  if (bars->abort_flag) return;
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
        int m_blk, n_blk, dst;
        tile_coords(p, t, m_blk, n_blk, dst);
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag);
          const uint32_t full = smem_u32(&bars->full[s]);
          mbar_arrive_expect_tx(full, STAGE_BYTES);
          const uint32_t a_dst = base + s * STAGE_BYTES;
          tma_load_2d(a_dst, &tm_a, full, kb * BK, m_blk * BM);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(a_dst + A_BYTES + j * B_BLOCK_BYTES, &tm_b, full, n_blk * BN + j * 64, kb * BK);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, BM, BN, 0, 1);
      uint32_t it = 0, local = 0;
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1u;
        mbar_wait(smem_u32(&bars->acc_empty[acc]), ((local >> 1) & 1u) ^ 1u, abort_flag);
        tc_fence_after();
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          mbar_wait(smem_u32(&bars->full[s]), (it / STAGES) & 1u, abort_flag);
          tc_fence_after();
          const uint32_t a_s = base + s * STAGE_BYTES;
          const uint32_t b_s = a_s + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = smem_desc_sw128(a_s + k * 32, 16, 1024);
            const uint64_t bd = smem_desc_sw128(b_s + k * 2048, B_BLOCK_BYTES, 1024);
            umma_f16_ss(tmem + acc * BN, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars->empty[s]));     // stage free once these MMAs have read it
        }
        umma_commit(smem_u32(&bars->acc_full[acc]));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2-5)
    const int lg = warp & 3;                         // TMEM lane group this warp may read
    const uint32_t stg = staging + lg * 8192;        // this warp's two 4 KB staging boxes
    uint32_t local = 0, box_it = 0;
    unsigned int* pending_flag = nullptr;            // lane 0: counter of the last remote tile, not yet released
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++local) {
      int m_blk, n_blk, dst;
      tile_coords(p, t, m_blk, n_blk, dst);
      const uint32_t acc = local & 1u;
      const int row = m_blk * BM + lg * 32 + lane;
      const bool remote = p.tp > 1 && dst != p.rank;
      if (remote) {
        // Before the first store into dst's receive slot make sure dst has consumed the previous
        // call's data (its done[] word, written by dst into this rank's flag buffer).
        if (lane == 0) {
          const unsigned int* done = p.flags[p.rank] + p.tp * p.blocks_per_shard + dst;
          if (ld_acquire_sys(done) + 1u < p.epoch && !*abort_flag) {
            const long long t0 = clock64();
            while (ld_acquire_sys(done) + 1u < p.epoch) {
              if (*abort_flag) break;
              if (clock64() - t0 > kWaitLimitCycles) { *abort_flag = 1; break; }
            }
          }
        }
        __syncwarp();
      } else if (p.tp > 1) {
        // Own rows: every other rank's partial tile must have landed in this rank's receive slots.
        if (lane == 0) {
          // Never enter this wait while holding back a release of our own (peers wait for it too).
          if (pending_flag != nullptr) {
            bulk_wait_all();
            fence_proxy_async_smem();
            __threadfence_system();
            red_release_sys_add(pending_flag, 1u);
            pending_flag = nullptr;
          }
          const int blk = m_blk - dst * p.blocks_per_shard;
          for (int src = 0; src < p.tp; ++src) {
            if (src == p.rank) continue;
            const unsigned int* f = p.flags[p.rank] + src * p.blocks_per_shard + blk;
            if (ld_acquire_sys(f) < p.flag_target && !*abort_flag) {
              const long long t0 = clock64();
              while (ld_acquire_sys(f) < p.flag_target) {
                if (*abort_flag) break;
                if (clock64() - t0 > kWaitLimitCycles) { *abort_flag = 1; break; }
              }
            }
          }
        }
        __syncwarp();
      }
      mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1u, abort_flag);
      tc_fence_after();

      if (remote) {
        // bf16 partial tile -> swizzled staging box -> TMA store into the owner's receive slot.
        const int y = (m_blk - dst * p.blocks_per_shard) * BM + lg * 32;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64, ++box_it) {
          const uint32_t buf = stg + (box_it & 1u) * 4096;
          if (lane == 0) bulk_wait_read1();          // the store that last used this buffer has read it
          __syncwarp();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t v[32];
            tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c0 + hh * 32), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int ch = hh * 4 + (j >> 3);
              const uint32_t d = buf + lane * 128 + ((ch ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d),
                           "r"(pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]))),
                           "r"(pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]))),
                           "r"(pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]))),
                           "r"(pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])))
                           : "memory");
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_out.m[dst], buf, n_blk * BN + c0, y);
            bulk_commit();
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bars->acc_empty[acc]));
          // Publish the PREVIOUS remote tile of this warp: its 4 store groups are older than the 4
          // just committed, so "at most 4 groups pending" means they have completed.  The owner
          // counts 4 arrivals (warps) per tile.
          if (pending_flag != nullptr) {
            bulk_wait_pending4();
            fence_proxy_async_smem();
            __threadfence_system();
            red_release_sys_add(pending_flag, 1u);
          }
          const int blk = m_blk - dst * p.blocks_per_shard;
          pending_flag = p.flags[dst] + p.rank * p.blocks_per_shard + blk;
        }
        __syncwarp();
      } else {
        __nv_bfloat16* orow;
        const __nv_bfloat16* rrow = nullptr;
        long long slot = 0;
        if (p.tp <= 1) {
          orow = p.c + static_cast<long long>(row) * p.ldc + n_blk * BN;
        } else {
          const int rl = row - dst * p.shard_rows;
          orow = p.out + static_cast<long long>(rl) * p.ldo + n_blk * BN;
          rrow = p.recv[p.rank] + static_cast<long long>(rl) * p.n + n_blk * BN;
          slot = static_cast<long long>(p.shard_rows) * p.n;
        }
        const bool row_ok = row < p.m;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c0), v);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n_blk * BN + c0 + j;
              if (col < p.n) {   // n is a multiple of 8
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[j + e]);
                if (rrow != nullptr) {
                  // fixed-order cross-rank sum: own fp32 accumulator, then sources 0..tp-1
                  for (int src = 0; src < p.tp; ++src) {
                    if (src == p.rank) continue;
                    const uint4 w = *reinterpret_cast<const uint4*>(rrow + src * slot + c0 + j);
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 ff = __bfloat1622float2(h2[e]);
                      f[2 * e] += ff.x;
                      f[2 * e + 1] += ff.y;
                    }
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(orow + c0 + j) = o;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
      }
    }
    if (lane == 0) {
      bulk_wait_all();
      if (pending_flag != nullptr) {
        fence_proxy_async_smem();
        __threadfence_system();
        red_release_sys_add(pending_flag, 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && p.status != nullptr && bars->abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
  if (tid == 0 && p.tp > 1) {
    // The last CTA to finish tells every peer that this rank's receive slots may be overwritten.
    __threadfence();
    const unsigned int prev = atomicAdd(p.counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.counter = 0;
      for (int peer = 0; peer < p.tp; ++peer)
        st_release_sys(p.flags[peer] + p.tp * p.blocks_per_shard + p.rank, p.epoch);
    }
  }
}

}  // namespace gemm
}  // namespace ftb

// ------------------------------------------------------------------------------------- host side
using namespace ftb;

static int launch_gemm(const void* a, const void* b, int m, int n, int k, long long lda, long long ldb,
                       gemm::Params& p, const gemm::OutMaps& maps, cudaStream_t st) {
  if (m <= 0 || n <= 0 || k <= 0) { set_last_error("gemm: bad sizes m=%d n=%d k=%d", m, n, k); return FTB_ERR_INVALID; }
  if ((n % 8) || (k % 8) || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(a) & 15) ||
      (reinterpret_cast<uintptr_t>(b) & 15)) {
    set_last_error("gemm: n, k and the leading dimensions must be multiples of 8 and pointers 16-byte aligned");
    return FTB_ERR_INVALID;
  }
  CUtensorMap tm_a, tm_b;
  if (!make_tmap_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, m, k, lda, gemm::BM, gemm::BK) ||
      !make_tmap_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, n, ldb, gemm::BK, 64)) {
    set_last_error("gemm: cuTensorMapEncodeTiled failed");
    return FTB_ERR_CUDA;
  }
  p.m = m; p.n = n; p.k = k;
  p.m_blocks = (m + gemm::BM - 1) / gemm::BM;
  p.n_blocks = (n + gemm::BN - 1) / gemm::BN;
  p.n_tiles = p.m_blocks * p.n_blocks;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.n_tiles < sms ? p.n_tiles : sms;
  cudaError_t e = cudaFuncSetAttribute(gemm::gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm)");
  gemm::gemm_bf16_kernel<<<grid, gemm::THREADS, gemm::SMEM_BYTES, st>>>(tm_a, tm_b, maps, p);
  return check_cuda(cudaGetLastError(), "gemm launch");
}

extern "C" FTB_API int ftb_gemm_bf16(const ftb_gemm_args* g, void* stream) {
  if (g == nullptr || !g->a || !g->b || !g->c) { set_last_error("ftb_gemm_bf16: null pointer"); return FTB_ERR_INVALID; }
  if ((g->ldc % 8) || (reinterpret_cast<uintptr_t>(g->c) & 15)) {
    set_last_error("ftb_gemm_bf16: c must be 16-byte aligned with ldc a multiple of 8");
    return FTB_ERR_INVALID;
  }
  gemm::Params p;
  memset(&p, 0, sizeof(p));
  p.c = reinterpret_cast<__nv_bfloat16*>(g->c);
  p.ldc = g->ldc;
  p.tp = 1;
  p.status = g->status;
  static gemm::OutMaps no_maps;   // unused when tp == 1
  return launch_gemm(g->a, g->b, g->m, g->n, g->k, g->lda, g->ldb, p, no_maps, reinterpret_cast<cudaStream_t>(stream));
}

struct ftb_gemm_rs_ctx {
  int rank, tp, m, n, shard_rows, blocks_per_shard;
  void* recv[gemm::MAX_TP];
  unsigned int* flags[gemm::MAX_TP];
  unsigned int* d_counter;
  unsigned int epoch;
  gemm::OutMaps maps;            // TMA store maps: receive slot of this rank on every peer
};

extern "C" FTB_API int ftb_gemm_rs_workspace_bytes(int m, int n, int tp, int64_t* recv_bytes, int64_t* flag_bytes) {
  if (m <= 0 || n <= 0 || tp <= 0 || tp > gemm::MAX_TP || (m % (tp * gemm::BM)) || (n % 8) || !recv_bytes || !flag_bytes) {
    set_last_error("ftb_gemm_rs_workspace_bytes: need 1 <= tp <= 8, m a multiple of tp*128, n a multiple of 8");
    return FTB_ERR_INVALID;
  }
  *recv_bytes = static_cast<int64_t>(m) * n * 2;                       // tp slots of [m/tp, n] bf16
  const int bps = m / tp / gemm::BM;
  *flag_bytes = static_cast<int64_t>(tp) * bps * 4 + tp * 4;           // tile counters + done words
  *flag_bytes = (*flag_bytes + 255) / 256 * 256;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs_ctx_create(ftb_gemm_rs_ctx** out, int rank, int tp, int m, int n,
                                              void* const* recv_ptrs, void* const* flag_ptrs) {
  int64_t rb, fb;
  if (!out || !recv_ptrs || !flag_ptrs || rank < 0 || rank >= tp) { set_last_error("ftb_gemm_rs_ctx_create: bad argument"); return FTB_ERR_INVALID; }
  int rc = ftb_gemm_rs_workspace_bytes(m, n, tp, &rb, &fb);
  if (rc != FTB_OK) return rc;
  ftb_gemm_rs_ctx* c = new ftb_gemm_rs_ctx();
  c->rank = rank; c->tp = tp; c->m = m; c->n = n;
  c->shard_rows = m / tp;
  c->blocks_per_shard = c->shard_rows / gemm::BM;
  c->epoch = 0;
  for (int i = 0; i < tp; ++i) {
    if (!recv_ptrs[i] || !flag_ptrs[i]) { delete c; set_last_error("ftb_gemm_rs_ctx_create: null peer pointer"); return FTB_ERR_INVALID; }
    c->recv[i] = recv_ptrs[i];
    c->flags[i] = reinterpret_cast<unsigned int*>(flag_ptrs[i]);
  }
  memset(&c->maps, 0, sizeof(c->maps));
  for (int i = 0; i < tp; ++i) {
    const char* slot = reinterpret_cast<const char*>(c->recv[i]) + static_cast<size_t>(rank) * c->shard_rows * n * 2;
    if (!make_tmap_2d(&c->maps.m[i], slot, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c->shard_rows, n, n, 32, 64)) {
      delete c;
      set_last_error("ftb_gemm_rs_ctx_create: cuTensorMapEncodeTiled failed for the receive slot of rank %d", i);
      return FTB_ERR_CUDA;
    }
  }
  cudaError_t e = cudaMalloc(&c->d_counter, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(c->d_counter, 0, sizeof(unsigned int));
  if (e != cudaSuccess) { delete c; return check_cuda(e, "ftb_gemm_rs_ctx_create"); }
  *out = c;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs_ctx_destroy(ftb_gemm_rs_ctx* c) {
  if (!c) return FTB_OK;
  cudaFree(c->d_counter);
  delete c;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs(ftb_gemm_rs_ctx* c, const void* a, const void* b, void* out, int k_local,
                                   int64_t lda, int64_t ldb, int64_t ldo, int32_t* status, void* stream) {
  if (!c || !a || !b || !out) { set_last_error("ftb_gemm_rs: null pointer"); return FTB_ERR_INVALID; }
  if ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) { set_last_error("ftb_gemm_rs: out alignment"); return FTB_ERR_INVALID; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  c->epoch += 1;
  gemm::Params p;
  memset(&p, 0, sizeof(p));
  p.tp = c->tp; p.rank = c->rank; p.shard_rows = c->shard_rows; p.blocks_per_shard = c->blocks_per_shard;
  for (int i = 0; i < c->tp; ++i) {
    p.recv[i] = reinterpret_cast<__nv_bfloat16*>(c->recv[i]);
    p.flags[i] = c->flags[i];
  }
  p.epoch = c->epoch;
  const int n_blocks = (c->n + gemm::BN - 1) / gemm::BN;
  p.flag_target = c->epoch * static_cast<unsigned int>(n_blocks) * 4u;   // 4 epilogue warps per tile
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.counter = c->d_counter;
  p.status = status;
  return launch_gemm(a, b, c->m, c->n, k_local, lda, ldb, p, c->maps, st);
}

// ---- CUDA IPC helpers for callers that do not have a symmetric-memory allocator of their own.
extern "C" FTB_API int ftb_ipc_alloc(int64_t bytes, void** ptr, uint8_t handle[64]) {
  if (!ptr || !handle || bytes <= 0) { set_last_error("ftb_ipc_alloc: bad argument"); return FTB_ERR_INVALID; }
  cudaError_t e = cudaMalloc(ptr, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return check_cuda(e, "ftb_ipc_alloc: cudaMalloc");
  e = cudaMemset(*ptr, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return check_cuda(e, "ftb_ipc_alloc: cudaMemset");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return check_cuda(e, "ftb_ipc_alloc: cudaIpcGetMemHandle");
  memcpy(handle, &h, 64);
  return FTB_OK;
}
extern "C" FTB_API int ftb_ipc_open(const uint8_t handle[64], void** ptr) {
  if (!ptr || !handle) { set_last_error("ftb_ipc_open: bad argument"); return FTB_ERR_INVALID; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "ftb_ipc_open");
}
extern "C" FTB_API int ftb_ipc_close(void* ptr) { return check_cuda(cudaIpcCloseMemHandle(ptr), "ftb_ipc_close"); }
extern "C" FTB_API int ftb_ipc_free(void* ptr) { return check_cuda(cudaFree(ptr), "ftb_ipc_free"); }
