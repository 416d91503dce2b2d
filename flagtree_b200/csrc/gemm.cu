// Persistent, warp-specialised tcgen05 GEMM for sm_100a: C[M,N] = A[M,K] . B[K,N], bf16 in, fp32
// accumulate in TMEM, bf16 out -- and the same kernel with a reduce-scatter epilogue: a finished tile
// whose rows belong to another rank is stored (bulk shared->global copies of contiguous 4 KB boxes, never a
// multicast load) straight into that rank's receive slot in peer memory over NVLink and a per-(source, row block)
// counter is released; tiles of this rank's own rows are computed last and their epilogue adds the
// partials the other ranks have pushed (fixed order, fp32) before writing the bf16 shard.
//
// Reduce-scatter by pull (used when the workspace has an NVSwitch multicast mapping): every rank writes
// its bf16 partial tiles into its OWN symmetric buffer, row blocks are visited in the same order on every
// rank, and when a row block is complete on a rank it raises one flag on the block's owner.  Four extra
// "reducer" warps per CTA wait for a row block's flags from all ranks and fetch the cross-rank sum with
// multimem.ld_reduce (in-switch reduction, fp32 accumulation): the owner's link carries 1/tp of the
// bytes and no SM ever pushes bulk data, so the MMA pipeline is not disturbed.
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

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int MAX_STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;                 // 16384
constexpr int B_BLOCK_BYTES = BK * 128;              // 8192: 64 k-rows x 64 columns
constexpr int STAGING_BYTES = 4 /*warps*/ * 2 /*buffers*/ * 4096;   // [32 rows x 128 B] boxes for bulk stores
// NCTA = 1: one CTA per 128 x 256 tile, it loads all of B (4 blocks), 4 stages of 48 KB.
// NCTA = 2: a CTA pair per 256 x 256 tile (cta_group::2 MMA); each CTA loads its 128 rows of A and
//           its 128 columns of B (2 blocks), 6 stages of 32 KB: a third less L2->SM traffic per flop.
template <int NCTA> struct Cfg {
  static constexpr int B_BLOCKS = (BN / 64) / NCTA;
  static constexpr int B_BYTES = B_BLOCKS * B_BLOCK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = NCTA == 1 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};
constexpr int THREADS = 192;
constexpr int THREADS_PULL = 320;      // + 4 reducer warps
constexpr int MAX_TP = 8;

struct Params {
  int m, n, k;
  int n_blocks, m_blocks, n_tiles;
  // The tiles of the last, partial wave are cut into two halves of 128 columns each so that twice as many CTA
  // groups share them: loop positions below n_full are whole tiles, the rest are halves (n_steps positions in all).
  int n_full, n_steps;
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
  // pull mode
  const __nv_bfloat16* mc_part;      // multicast address of the ranks' partial buffers [m, n] (NULL = push mode)
  unsigned int* blk_counter;         // per 128-row block: epilogue-warp arrivals, monotonic over calls
  long long wait_limit;              // cycles after which a wait for another rank gives up (status = timeout)
  // copy-engine exchange: every tile is stored into the local partial (c / ldc); when the last tile of a row
  // shard has been stored its word in ce_ready takes the call number, which a stream memory operation waits for
  // Row shards leave in ce_chunks pieces of consecutive row blocks each (words [d * ce_chunks + piece]); the peers'
  // pieces of this rank's own rows arrive in its receive slots (row-major [tp][shard_rows][n]) with a flag per
  // (source, piece), and the epilogue of the own rows, which come last, adds them: no separate reduce pass.
  unsigned int* ce_ready;            // [tp * ce_chunks] (NULL = another protocol)
  unsigned int* ce_cnt;              // [tp * ce_chunks] epilogue-warp arrivals per piece, monotonic over calls
  unsigned int ce_target[8];         // value ce_cnt[d * ce_chunks + piece] reaches in this call (pieces may differ in size)
  int ce_chunks;                     // <= 8
  int ce_groups, ce_group_blocks;    // row groups per shard, row blocks per group (2 when the shard has an even number)
  // all-gather + GEMM: the rows of A arrive shard by shard (copy engines of the peers); ag_flags[src] takes the
  // call number once rank src's shard is in place.  NULL = A is complete at launch.  The rank's own rows are read
  // from the caller's shard through a tensor map of their own (no copy, no wait).
  const unsigned int* ag_flags;
};


// SS-form MMA (one CTA or a pair) with the descriptors as 32-bit halves and a compile-time accumulate flag
template <int NCTA, bool kAccumulate>
__device__ __forceinline__ void umma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc) {
  if constexpr (NCTA == 1) {
    umma_f16_ss_lohi<kAccumulate>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc);
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 ad, bd;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 ad, {%1, %2};\n\t"
        "mov.b64 bd, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], ad, bd, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
  }
}

struct Bars {
  unsigned long long full[MAX_STAGES];
  unsigned long long empty[MAX_STAGES];
  unsigned long long acc_full[2];
  unsigned long long acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Tile t of a CTA group (NCTA CTAs, each owning one 128-row block of the group tile) -> the 128-row
// block of CTA `cta`, the 256-column block, and the rank that owns those rows.
template <int NCTA, bool PULL = false>
__device__ __forceinline__ void tile_coords(const Params& p, int t, int cta, int& m_blk, int& n_blk, int& dst) {
  if constexpr (PULL) {
    // row-block group j of every shard (shards staggered by rank), then group j+1 ...: row block j of
    // every owner is complete on all ranks after phase j, so owners can fetch while phase j+1 runs.
    const int per_phase = p.tp * p.n_blocks;
    const int jg = t / per_phase;
    const int r = t - jg * per_phase;
    const int so = r / p.n_blocks;
    n_blk = r - so * p.n_blocks;
    dst = (so + p.rank) % p.tp;
    m_blk = dst * p.blocks_per_shard + jg * NCTA + cta;
    return;
  }
  if (p.tp <= 1) {
    const int mg = t / p.n_blocks;
    n_blk = t - mg * p.n_blocks;
    m_blk = mg * NCTA + cta;
    dst = 0;
    return;
  }
  const int groups_per_shard = p.blocks_per_shard / NCTA;
  const int per_shard = groups_per_shard * p.n_blocks;
  const int ord = t / per_shard;
  // reduce-scatter: remote shards first, own shard last.  All-gather: own rows first, then the shard of rank - 1
  // (every rank sends to rank + 1 first), rank - 2, ...
  dst = p.ag_flags != nullptr ? (p.rank - ord + p.tp) % p.tp : (p.rank + 1 + ord) % p.tp;
  const int r = t - ord * per_shard;
  const int mg = r / p.n_blocks;
  n_blk = r - mg * p.n_blocks;
  m_blk = dst * p.blocks_per_shard + mg * NCTA + cta;
}

// Loop position -> tile number, first column of the tile that this step computes, and its width.
struct Step { int tile, col_off, width; };
__device__ __forceinline__ Step step_of(const Params& p, int pos) {
  if (pos < p.n_full) return Step{pos, 0, BN};
  const int r = pos - p.n_full;
  return Step{p.n_full + (r >> 1), (r & 1) * (BN / 2), BN / 2};
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

// 4 KB contiguous shared -> global copy (the destination may be peer memory).
__device__ __forceinline__ void bulk_store_4k(void* dst, uint32_t src) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 4096;" ::"l"(dst), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_pending4() { asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Epilogue of a tile whose rows this rank owns: out = own fp32 accumulator + partials of the other
// ranks (ascending rank order, fp32), as bf16.  The partials are fetched with two 16-column slices in
// flight per thread (NSRC x 2 16-byte loads each) and the first slice is requested before the
// accumulator is complete, so the load latency overlaps the MMAs.  NSRC = tp - 1 (0 = generic path).
template <int NSRC>
__device__ __forceinline__ void own_tile_epilogue(const Params& p, int rl, long long slot,
                                                  __nv_bfloat16* orow, int n_blk, uint32_t full_bar, uint32_t parity,
                                                  uint32_t tacc, volatile int* abort_flag, bool skip_reads,
                                                  int col_off, int width, bool row_major) {
  const int col_base = n_blk * BN + col_off;          // first column of this step; `orow` points at it
  constexpr int NS = NSRC > 0 ? NSRC : 1;
  // Receive slots are stored as contiguous 4 KB boxes of [32 rows x 64 columns] in the staging
  // (128B-swizzled) order; `rrow` points at this thread's row inside box column 0 of its row group.
  // With the copy-engine exchange the slots are plain row-major [shard_rows][n].
  const __nv_bfloat16* rrow = row_major ? p.recv[p.rank] + static_cast<long long>(rl) * p.n
                                        : p.recv[p.rank] + static_cast<long long>(rl >> 5) * (p.n >> 6) * 2048 + (rl & 31) * 64;
  const int sw = rl & 7;
  auto box_off = [&](int col) -> long long {   // element offset of 8 columns starting at absolute column `col`
    return row_major ? static_cast<long long>(col)
                     : static_cast<long long>(col >> 6) * 2048 + ((((col & 63) >> 3) ^ sw) << 3);
  };
  const __nv_bfloat16* src_ptr[NS];
  if constexpr (NSRC > 0) {
#pragma unroll
    for (int i = 0; i < NSRC; ++i) src_ptr[i] = rrow + (i + (i >= p.rank ? 1 : 0)) * slot;   // ascending, skipping self
  }
  uint4 bufA[NS][2], bufB[NS][2];
  auto fetch = [&](uint4 (&buf)[NS][2], int col) {
    if constexpr (NSRC > 0) {
      if (!skip_reads && col_base + col < p.n) {
#pragma unroll
        for (int i = 0; i < NSRC; ++i) {
          buf[i][0] = *reinterpret_cast<const uint4*>(src_ptr[i] + box_off(col_base + col));
          buf[i][1] = *reinterpret_cast<const uint4*>(src_ptr[i] + box_off(col_base + col + 8));
        }
      } else {
#pragma unroll
        for (int i = 0; i < NSRC; ++i) buf[i][0] = buf[i][1] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto finish = [&](const uint32_t* v, uint4 (&buf)[NS][2], int col) {
    float f[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[e]);
    if constexpr (NSRC > 0) {
#pragma unroll
      for (int i = 0; i < NSRC; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&buf[i][h]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 ff = __bfloat1622float2(h2[e]);
            f[h * 8 + 2 * e] += ff.x;
            f[h * 8 + 2 * e + 1] += ff.y;
          }
        }
      }
    } else if (!skip_reads && col_base + col < p.n) {
      for (int src = 0; src < p.tp; ++src) {
        if (src == p.rank) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 w = *reinterpret_cast<const uint4*>(rrow + src * slot + box_off(col_base + col + h * 8));
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 ff = __bfloat1622float2(h2[e]);
            f[h * 8 + 2 * e] += ff.x;
            f[h * 8 + 2 * e + 1] += ff.y;
          }
        }
      }
    }
    if (col_base + col < p.n) {   // n is a multiple of 8 (and row blocks are full in this mode)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (col_base + col + h * 8 < p.n) {
          uint4 o;
          o.x = pack_bf16x2(f[h * 8], f[h * 8 + 1]);
          o.y = pack_bf16x2(f[h * 8 + 2], f[h * 8 + 3]);
          o.z = pack_bf16x2(f[h * 8 + 4], f[h * 8 + 5]);
          o.w = pack_bf16x2(f[h * 8 + 6], f[h * 8 + 7]);
          *reinterpret_cast<uint4*>(orow + col + h * 8) = o;
        }
      }
    }
  };
  fetch(bufA, 0);
  if (!__all_sync(0xffffffffu, mbar_wait(full_bar, parity, abort_flag))) return;   // a wait ran out: the tile is not written
  tc_fence_after();
#pragma unroll 1
  for (int c0 = 0; c0 < width; c0 += 32) {
    fetch(bufB, c0 + 16);
    uint32_t v[32];
    tmem_ld32(tacc + c0, v);
    tmem_wait_ld();
    finish(v, bufA, c0);
    if (c0 + 32 < width) fetch(bufA, c0 + 32);
    finish(v + 16, bufB, c0 + 16);
  }
}

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr));
  return v;
}

template <int NCTA, bool PULL>
__global__ void __launch_bounds__(PULL ? THREADS_PULL : THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_a_own, const Params p) {
  using C = Cfg<NCTA>;
  constexpr int STAGES = C::STAGES;
  constexpr int STAGE_BYTES = C::STAGE_BYTES;
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
  const int cta = NCTA == 1 ? 0 : static_cast<int>(cluster_ctarank());   // position inside the CTA pair
  const int group = blockIdx.x / NCTA;
  const int n_groups = gridDim.x / NCTA;

  if (tid == 0) {
    bars->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->acc_full[a]), 1);
      mbar_init(smem_u32(&bars->acc_empty[a]), 4 * NCTA);   // one arrival per epilogue warp of the group
    }
    fence_mbar_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_a_own);
    tma_prefetch_desc(&tm_b);
  }
  __syncthreads();
  // An earlier launch on this status word failed: leave at once.  The two CTAs of a pair read the word at
  // different moments (another group of this launch may report a timeout in between), so the odd CTA takes the
  // even CTA's reading: a CTA that went on alone would signal barriers in the shared memory of a partner that
  // has left.
  if constexpr (NCTA == 2) {
    cluster_sync_all();
    uint32_t leave;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(leave) : "r"(mapa_shared(smem_u32(&bars->abort_flag), 0)) : "memory");
    cluster_sync_all();        // the even CTA keeps its flag until its partner has read it
    if (tid == 0) bars->abort_flag = leave != 0u ? 1 : 0;
    __syncthreads();
  }
  if (bars->abort_flag) {
    // copy-engine exchange: the second stream waits for the ready words whatever became of this launch
    if (p.ce_ready != nullptr && blockIdx.x == 0 && tid < p.tp * p.ce_chunks) st_release_sys(p.ce_ready + tid, p.epoch);
    return;   // (an all-gather launch that leaves here does not release the peers: the context is dead)
  }
  if (warp == 1) {
    if constexpr (NCTA == 1) {
      tmem_alloc(smem_u32(&bars->tmem_base), 512);
      tmem_relinquish();
    } else {
      tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
      tmem_relinquish_pair();
    }
    tc_fence_before();
  }
  __syncthreads();
  if constexpr (NCTA == 2) cluster_sync_all();   // peer barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (every CTA)
    if (lane == 0) {
      uint32_t it = 0;
      for (int pos = group; pos < p.n_steps; pos += n_groups) {
        const Step stp = step_of(p, pos);
        int m_blk, n_blk, dst;
        tile_coords<NCTA, PULL>(p, stp.tile, cta, m_blk, n_blk, dst);
        const int b_blocks = stp.width / 64 / NCTA;          // 64-column blocks of B this CTA loads per stage
        const int b_col0 = n_blk * BN + stp.col_off + cta * b_blocks * 64;
        const uint32_t stage_tx = A_BYTES + b_blocks * B_BLOCK_BYTES;
        const bool own_rows = p.ag_flags != nullptr && dst == p.rank;
        const CUtensorMap* ta = own_rows ? &tm_a_own : &tm_a;
        const int a_row0 = own_rows ? m_blk * BM - p.rank * p.shard_rows : m_blk * BM;
        if (p.ag_flags != nullptr && !own_rows && ld_acquire_sys(p.ag_flags + dst) < p.epoch && !*abort_flag) {
          // all-gather: the rows of this tile come from rank dst; wait (bounded) until its copy has landed
          const long long t0 = clock64();
          while (ld_acquire_sys(p.ag_flags + dst) < p.epoch) {
            if (*abort_flag) break;
            if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; break; }
            __nanosleep(200);
          }
        }
        // the copy was seen through the generic proxy, the loads below use the async one
        if (p.ag_flags != nullptr) asm volatile("fence.proxy.async;" ::: "memory");
        if (*abort_flag) break;                              // a wait ran out: nothing more is loaded
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag)) break;
          const uint32_t a_dst = base + s * STAGE_BYTES;
          if constexpr (NCTA == 1) {
            const uint32_t full = smem_u32(&bars->full[s]);
            mbar_arrive_expect_tx(full, stage_tx);
            tma_load_2d(a_dst, ta, full, kb * BK, a_row0);
#pragma unroll
            for (int j = 0; j < C::B_BLOCKS; ++j)
              if (j < b_blocks) tma_load_2d(a_dst + A_BYTES + j * B_BLOCK_BYTES, &tm_b, full, b_col0 + j * 64, kb * BK);
          } else {
            // Both CTAs' loads are counted on the even CTA's barrier; that CTA announces the total.
            const uint32_t full0 = mapa_shared(smem_u32(&bars->full[s]), 0);
            if (cta == 0) mbar_arrive_expect_tx(smem_u32(&bars->full[s]), 2 * stage_tx);
            tma_load_2d_pair(a_dst, ta, full0, kb * BK, a_row0);
#pragma unroll
            for (int j = 0; j < C::B_BLOCKS; ++j)
              if (j < b_blocks) tma_load_2d_pair(a_dst + A_BYTES + j * B_BLOCK_BYTES, &tm_b, full0, b_col0 + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    // The whole warp runs the loop and waits; an elected lane (always the same one, so that its commits cover
    // its MMAs) issues.  Descriptors: only the low word (address) changes, by constants per k step.
    if (cta == 0) {
      constexpr uint32_t kIdescFull = umma_idesc(kFmtBF16, BM * NCTA, BN, 0, 1);
      constexpr uint32_t kIdescHalf = umma_idesc(kFmtBF16, BM * NCTA, BN / 2, 0, 1);
      const uint64_t ad0 = smem_desc_sw128(base, 16, 1024);
      const uint64_t bd0 = smem_desc_sw128(base + A_BYTES, B_BLOCK_BYTES, 1024);
      const uint32_t ad_lo0 = static_cast<uint32_t>(ad0), ad_hi = static_cast<uint32_t>(ad0 >> 32);
      const uint32_t bd_lo0 = static_cast<uint32_t>(bd0), bd_hi = static_cast<uint32_t>(bd0 >> 32);
      const uint32_t full0 = smem_u32(&bars->full[0]);
      const uint32_t empty_own = NCTA == 1 ? smem_u32(&bars->empty[0]) : mapa_shared(smem_u32(&bars->empty[0]), 0);
      const uint32_t empty_peer = NCTA == 1 ? 0u : mapa_shared(smem_u32(&bars->empty[0]), 1);
      const uint32_t accf_own = NCTA == 1 ? smem_u32(&bars->acc_full[0]) : mapa_shared(smem_u32(&bars->acc_full[0]), 0);
      const uint32_t accf_peer = NCTA == 1 ? 0u : mapa_shared(smem_u32(&bars->acc_full[0]), 1);
      uint32_t s = 0, ph = 0, local = 0;     // stage and its phase bit, tiles done by this group
      for (int pos = group; pos < p.n_steps; pos += n_groups, ++local) {
        const uint32_t kIdesc = pos < p.n_full ? kIdescFull : kIdescHalf;
        const uint32_t acc = local & 1u;
        // a wait that ran out ends the loop for the whole warp: no more MMAs
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_empty[acc]), ((local >> 1) & 1u) ^ 1u, abort_flag))) break;
        tc_fence_after();
        const uint32_t d = tmem + acc * BN;
        bool live = true;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(full0 + s * 8, ph, abort_flag))) { live = false; break; }
          tc_fence_after();
          const uint32_t a_lo = ad_lo0 + ((s * STAGE_BYTES) >> 4);
          const uint32_t b_lo = bd_lo0 + ((s * STAGE_BYTES) >> 4);
          if (elect_one()) {
            if (kb == 0) {
              umma_ss_lohi<NCTA, false>(d, a_lo, ad_hi, b_lo, bd_hi, kIdesc);
#pragma unroll
              for (int k = 1; k < BK / 16; ++k)
                umma_ss_lohi<NCTA, true>(d, a_lo + ((k * 32) >> 4), ad_hi, b_lo + ((k * 2048) >> 4), bd_hi, kIdesc);
            } else {
#pragma unroll
              for (int k = 0; k < BK / 16; ++k)
                umma_ss_lohi<NCTA, true>(d, a_lo + ((k * 32) >> 4), ad_hi, b_lo + ((k * 2048) >> 4), bd_hi, kIdesc);
            }
            // stage free (in every CTA of the group) once these MMAs have read it
            if constexpr (NCTA == 1) {
              umma_commit(empty_own + s * 8);
            } else {
              umma_commit_pair(empty_own + s * 8);
              umma_commit_pair(empty_peer + s * 8);
            }
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!live) break;
        if (elect_one()) {
          if constexpr (NCTA == 1) {
            umma_commit(accf_own + acc * 8);
          } else {
            umma_commit_pair(accf_own + acc * 8);
            umma_commit_pair(accf_peer + acc * 8);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2-5)
    const int lg = warp & 3;                         // TMEM lane group this warp may read
    const uint32_t stg = staging + lg * 8192;        // this warp's two 4 KB staging boxes
    uint32_t local = 0, box_it = 0;
    unsigned int* pending_flag = nullptr;            // lane 0: counter of the last remote tile, not yet released
    int ce_pending = -1;                             // lane 0, copy-engine exchange: row shard of the tile stored last, not yet counted
    unsigned int ce_weight = 0;                      // what that tile counts: 2 for a whole tile, 1 for a half
    int pull_pending_blk = -1;                       // lane 0, pull protocol: row block of the tile stored last, not yet counted
    unsigned int* pull_pending_flag = nullptr;       // the owner's word for that row block
    // the accumulator-free barrier the MMA issuer waits on lives in the even CTA
    const uint32_t acc_empty_addr[2] = {
        NCTA == 1 ? smem_u32(&bars->acc_empty[0]) : mapa_shared(smem_u32(&bars->acc_empty[0]), 0),
        NCTA == 1 ? smem_u32(&bars->acc_empty[1]) : mapa_shared(smem_u32(&bars->acc_empty[1]), 0)};
    auto release_acc = [&](uint32_t a) {
      if constexpr (NCTA == 1) mbar_arrive(acc_empty_addr[a]);
      else mbar_arrive_cluster(acc_empty_addr[a]);
    };
    for (int pos = group; pos < p.n_steps; pos += n_groups, ++local) {
      const Step stp = step_of(p, pos);
      int m_blk, n_blk, dst;
      tile_coords<NCTA, PULL>(p, stp.tile, cta, m_blk, n_blk, dst);
      const uint32_t acc = local & 1u;
      const int row = m_blk * BM + lg * 32 + lane;
      const bool ag = !PULL && p.ag_flags != nullptr;
      const bool ce_own = !PULL && p.ce_ready != nullptr && dst == p.rank;   // copy-engine exchange, own rows: reduced here
      const bool ce = !PULL && !ce_own && (p.ce_ready != nullptr || ag);    // tiles stored plainly into c
      const bool remote = !PULL && !ce && !ce_own && p.tp > 1 && dst != p.rank;
      const int blk_in_shard = m_blk - dst * p.blocks_per_shard;
      // row group g of a shard belongs to piece floor(g * pieces / groups)
      const int piece = p.ce_ready != nullptr ? (blk_in_shard / p.ce_group_blocks) * p.ce_chunks / p.ce_groups : 0;
      if constexpr (PULL) {
        // Before overwriting a row block of the partial buffer make sure its owner has fetched the
        // previous call's sum (the owner's done[] word in this rank's flag buffer).
        if (lane == 0) {
          const unsigned int* done = p.flags[p.rank] + p.tp * p.blocks_per_shard + dst;
          if (ld_acquire_sys(done) + 1u < p.epoch && !*abort_flag) {
            const long long t0 = clock64();
            while (ld_acquire_sys(done) + 1u < p.epoch) {
              if (*abort_flag) break;
              if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; break; }
            }
          }
        }
        __syncwarp();
      } else if (remote) {
        // Before the first store into dst's receive slot make sure dst has consumed the previous
        // call's data (its done[] word, written by dst into this rank's flag buffer).
        if (lane == 0) {
          const unsigned int* done = p.flags[p.rank] + p.tp * p.blocks_per_shard + dst;
          if (ld_acquire_sys(done) + 1u < p.epoch && !*abort_flag) {
            const long long t0 = clock64();
            while (ld_acquire_sys(done) + 1u < p.epoch) {
              if (*abort_flag) break;
              if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; break; }
            }
          }
        }
        __syncwarp();
      } else if (!PULL && !ce && p.tp > 1) {
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
          if (ce_pending >= 0) {
            __threadfence();
            const unsigned int cnt = atomicAdd(p.ce_cnt + ce_pending, ce_weight) + ce_weight;
            if (cnt == p.ce_target[ce_pending % p.ce_chunks]) st_release_sys(p.ce_ready + ce_pending, p.epoch);
            ce_pending = -1;
          }
          const int blk = m_blk - dst * p.blocks_per_shard;
          // push: a counter per (source, row block) that reaches flag_target; copy engines: a word per
          // (source, piece) that takes the call number
          const int words_per_src = ce_own ? p.ce_chunks : p.blocks_per_shard;
          const int word = ce_own ? piece : blk;
          const unsigned int want = ce_own ? p.epoch : p.flag_target;
          for (int src = 0; src < p.tp; ++src) {
            if (src == p.rank) continue;
            const unsigned int* f = p.flags[p.rank] + src * words_per_src + word;
            if (ld_acquire_sys(f) < want && !*abort_flag) {
              const long long t0 = clock64();
              while (ld_acquire_sys(f) < want) {
                if (*abort_flag) break;
                if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; break; }
              }
            }
          }
        }
        __syncwarp();
      }
      if constexpr (PULL) {
        // partial tile -> this rank's own symmetric buffer (row-major [m, n] bf16), then count the row block
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1u, abort_flag))) break;   // a wait ran out
        tc_fence_after();
        if (lane == 0 && pull_pending_blk >= 0) {
          // Count the tile stored BEFORE this one for its row block: its stores left a whole tile ago, so the fence
          // that orders them before the count returns at once (a system-scope fence right behind the stores of
          // every tile held the epilogue, and with it the MMAs, back).  The last count of a row block on this rank
          // tells the owner, with the one system-scope release that the peers' reads need.
          __threadfence();
          const unsigned int cnt = atomicAdd(p.blk_counter + pull_pending_blk, 1u) + 1u;
          if (cnt == p.flag_target) {
            __threadfence_system();
            st_release_sys(pull_pending_flag, p.epoch);
          }
          pull_pending_blk = -1;
        }
        __syncwarp();                  // the tensor-memory loads below are warp-collective
        __nv_bfloat16* orow = p.recv[p.rank] + static_cast<long long>(row) * p.n + n_blk * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c0), v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (n_blk * BN + c0 + j < p.n) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
              *reinterpret_cast<uint4*>(orow + c0 + j) = o;
            }
          }
        }
        tc_fence_before();
        __syncwarp();                  // orders the 32 lanes' stores before lane 0's fence below
        if (lane == 0) {
          release_acc(acc);
          const int blk = m_blk - dst * p.blocks_per_shard;
          pull_pending_blk = m_blk;    // counted one tile late, see above
          pull_pending_flag = p.flags[dst] + p.rank * p.blocks_per_shard + blk;
        }
        __syncwarp();
      } else if (remote) {
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1u, abort_flag))) break;   // a wait ran out
        tc_fence_after();
        // Drain the accumulator into registers as packed bf16 and hand the TMEM buffer back at once,
        // so that a slow link only delays this warp's stores, not the MMAs of the next tiles.
        uint32_t pk[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c * 32), v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[c * 16 + j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(acc);
        // packed registers -> swizzled staging box -> bulk store into the owner's receive slot.
        const int y = (m_blk - dst * p.blocks_per_shard) * BM + lg * 32;
#pragma unroll
        for (int bx = 0; bx < BN / 64; ++bx, ++box_it) {
          const uint32_t buf = stg + (box_it & 1u) * 4096;
          if (lane == 0) bulk_wait_read1();          // the store that last used this buffer has read it
          __syncwarp();
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t d = buf + lane * 128 + ((ch ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d), "r"(pk[bx * 32 + ch * 4]),
                         "r"(pk[bx * 32 + ch * 4 + 1]), "r"(pk[bx * 32 + ch * 4 + 2]), "r"(pk[bx * 32 + ch * 4 + 3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && n_blk * BN + bx * 64 < p.n) {
            __nv_bfloat16* box = p.recv[dst] + static_cast<long long>(p.rank) * p.shard_rows * p.n +
                                 (static_cast<long long>(y >> 5) * (p.n >> 6) + (n_blk * (BN / 64) + bx)) * 2048;
            bulk_store_4k(box, buf);
            bulk_commit();
          }
        }
        if (lane == 0) {
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
      } else if (!PULL && !ce && p.tp > 1) {
        const int rl = row - dst * p.shard_rows;
        __nv_bfloat16* orow = p.out + static_cast<long long>(rl) * p.ldo + n_blk * BN + stp.col_off;
        const long long slot = static_cast<long long>(p.shard_rows) * p.n;
        const uint32_t full_bar = smem_u32(&bars->acc_full[acc]);
        const uint32_t par = (local >> 1) & 1u;
        const uint32_t tacc = tmem_addr(tmem, lg * 32, acc * BN);
        const bool skip = false;
        switch (p.tp) {
          case 2: own_tile_epilogue<1>(p, rl, slot, orow, n_blk, full_bar, par, tacc, abort_flag, skip, stp.col_off, stp.width, ce_own); break;
          case 4: own_tile_epilogue<3>(p, rl, slot, orow, n_blk, full_bar, par, tacc, abort_flag, skip, stp.col_off, stp.width, ce_own); break;
          case 8: own_tile_epilogue<7>(p, rl, slot, orow, n_blk, full_bar, par, tacc, abort_flag, skip, stp.col_off, stp.width, ce_own); break;
          default: own_tile_epilogue<0>(p, rl, slot, orow, n_blk, full_bar, par, tacc, abort_flag, skip, stp.col_off, stp.width, ce_own); break;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(acc);
      } else if (!PULL) {
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1u, abort_flag))) break;   // a wait ran out
        tc_fence_after();
        if (ce && lane == 0 && ce_pending >= 0) {
          // Copy-engine exchange: count the tile stored BEFORE this one for its row shard.  Its stores left a
          // whole tile ago, so the fence that orders them before the count returns at once (a fence right behind
          // the stores of a tile cost the GEMM a quarter of its time); the copy engine and the stream wait read
          // through L2, so device scope is enough.  The last count of a shard publishes "shard complete".
          __threadfence();
          const unsigned int cnt = atomicAdd(p.ce_cnt + ce_pending, ce_weight) + ce_weight;
          if (cnt == p.ce_target[ce_pending % p.ce_chunks]) st_release_sys(p.ce_ready + ce_pending, p.epoch);
          ce_pending = -1;
        }
        __syncwarp();                  // the tensor-memory loads below are warp-collective
        __nv_bfloat16* orow = p.c + static_cast<long long>(row) * p.ldc + n_blk * BN + stp.col_off;
        const bool row_ok = row < p.m;
#pragma unroll 1
        for (int c0 = 0; c0 < stp.width; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_addr(tmem, lg * 32, acc * BN + c0), v);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n_blk * BN + stp.col_off + c0 + j;
              if (col < p.n) {   // n is a multiple of 8
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                *reinterpret_cast<uint4*>(orow + c0 + j) = o;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();                  // orders the 32 lanes' stores before lane 0's fence one tile later
        if (lane == 0) {
          release_acc(acc);
          if (ce && !ag) { ce_pending = dst * p.ce_chunks + piece; ce_weight = stp.width == BN ? 2u : 1u; }   // counted one tile late, see above
        }
      }
    }
    if (lane == 0 && pull_pending_blk >= 0) {
      __threadfence();
      const unsigned int cnt = atomicAdd(p.blk_counter + pull_pending_blk, 1u) + 1u;
      if (cnt == p.flag_target) {
        __threadfence_system();
        st_release_sys(pull_pending_flag, p.epoch);
      }
    }
    if (lane == 0 && ce_pending >= 0) {
      __threadfence();
      const unsigned int cnt = atomicAdd(p.ce_cnt + ce_pending, ce_weight) + ce_weight;
      if (cnt == p.ce_target[ce_pending % p.ce_chunks]) st_release_sys(p.ce_ready + ce_pending, p.epoch);
    }
    if (lane == 0) {
      bulk_wait_all();
      if (pending_flag != nullptr) {
        fence_proxy_async_smem();
        __threadfence_system();
        red_release_sys_add(pending_flag, 1u);
      }
    }
  } else {
    // ------------------------------------------------------------------ reducers (warps 6-9, pull mode)
    if constexpr (PULL) {
      const int rt = tid - 192;                      // 0..127
      const int vec_per_row = p.n >> 3;
      const int vec_per_blk = BM * vec_per_row;
      for (int j = 0; j < p.blocks_per_shard; ++j) {
        if (lane == 0) {
          for (int src = 0; src < p.tp; ++src) {
            const unsigned int* f = p.flags[p.rank] + src * p.blocks_per_shard + j;
            if (ld_acquire_sys(f) < p.epoch && !*abort_flag) {
              const long long t0 = clock64();
              while (ld_acquire_sys(f) < p.epoch) {
                if (*abort_flag) break;
                if (clock64() - t0 > p.wait_limit) { *abort_flag = 1; break; }
                __nanosleep(100);
              }
            }
          }
        }
        __syncwarp();
        if (*abort_flag) break;
        const long long row0 = static_cast<long long>(p.rank) * p.shard_rows + j * BM;
        const __nv_bfloat16* src_blk = p.mc_part + row0 * p.n;
        __nv_bfloat16* out_blk = p.out + static_cast<long long>(j) * BM * p.ldo;
        // 16 fetches in flight per thread: the sums come back over NVLink with microseconds of latency
        const int stride = gridDim.x * 128;
        for (int i0 = blockIdx.x * 128 + rt; i0 < vec_per_blk; i0 += 16 * stride) {
          uint4 v[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int i = i0 + u * stride;
            if (i < vec_per_blk) v[u] = multimem_ld_reduce_bf16x8(src_blk + static_cast<long long>(i) * 8);
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int i = i0 + u * stride;
            if (i < vec_per_blk) {
              const int r = i / vec_per_row;
              const int c = (i - r * vec_per_row) * 8;
              *reinterpret_cast<uint4*>(out_blk + static_cast<long long>(r) * p.ldo + c) = v[u];
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) {
    // A wait ran out somewhere in this CTA.  Loads that were already issued still land in this CTA's shared memory
    // and MMAs already issued still read it: give them time (bounded) before the CTA may leave.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    // copy-engine exchange: the second stream waits for the ready words whatever became of this launch
    if (p.ce_ready != nullptr && tid < p.tp * p.ce_chunks) st_release_sys(p.ce_ready + tid, p.epoch);
  }
  if constexpr (NCTA == 2) cluster_sync_all();   // no CTA leaves while its peer may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (NCTA == 1) tmem_dealloc(tmem, 512);
    else tmem_dealloc_pair(tmem, 512);
  }
  if (tid == 0 && p.status != nullptr && bars->abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
  if (tid == 0 && p.tp > 1) {
    // The last CTA to finish tells every peer that this rank's receive slots may be overwritten; with the
    // copy-engine exchange it raises this rank's own "partial complete" word for the reduce kernel instead.
    __threadfence();
    const unsigned int prev = atomicAdd(p.counter, 1u);
    if (prev == gridDim.x - 1) {   // every CTA of the launch has arrived
      *p.counter = 0;
      if (p.ag_flags != nullptr) {
        // all-gather: every peer may overwrite its shard in this rank's gather buffer
        for (int peer = 0; peer < p.tp; ++peer) st_release_sys(p.flags[peer] + p.tp + p.rank, p.epoch);
      } else if (p.ce_ready != nullptr) {
        // copy-engine exchange: the peers' pieces in this rank's receive slots have been read
        for (int peer = 0; peer < p.tp; ++peer) st_release_sys(p.flags[peer] + p.tp * p.ce_chunks + p.rank, p.epoch);
      } else {
        for (int peer = 0; peer < p.tp; ++peer)
          st_release_sys(p.flags[peer] + p.tp * p.blocks_per_shard + p.rank, p.epoch);
      }
    }
  }
}

}  // namespace gemm
}  // namespace ftb

// ------------------------------------------------------------------------------------- host side
using namespace ftb;

// Stream memory operations (driver entry points, looked up through the runtime like cuTensorMapEncodeTiled).
typedef CUresult (*StreamValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
static StreamValue32Fn get_stream_memop(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<StreamValue32Fn>(p);
  return nullptr;
}

template <int NCTA, bool PULL>
static int launch_variant(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_a_own, const gemm::Params& p, int sms,
                          cudaStream_t st) {
  auto kern = gemm::gemm_bf16_kernel<NCTA, PULL>;
  constexpr int smem = gemm::Cfg<NCTA>::SMEM_BYTES;
  constexpr int threads = PULL ? gemm::THREADS_PULL : gemm::THREADS;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm)");
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = NCTA; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int max_groups = sms / NCTA;
  if (NCTA == 2) {
    cfg.gridDim = dim3(2);
    int mc = 0;
    e = cudaOccupancyMaxActiveClusters(&mc, kern, &cfg);
    if (e == cudaSuccess && mc > 0) max_groups = mc; else cudaGetLastError();
  }
  // pull mode: every CTA must be resident at once (reducer warps wait on other CTAs' tiles): the
  // grid never exceeds one CTA per SM, which this kernel's shared-memory footprint already enforces.
  const int groups = p.n_tiles < max_groups ? p.n_tiles : max_groups;
  cfg.gridDim = dim3(NCTA * groups);
  // Tiles left over after the whole waves: when at most half of the groups would have one, each is cut into two
  // halves of 128 columns.  The push protocol sends whole tiles only, so there the leftover must lie in the
  // rank's own row shard (the last tiles of the order); the pull protocol keeps whole tiles.
  gemm::Params q = p;
  const int left = p.n_tiles % groups;
  const bool push = p.tp > 1 && p.ce_ready == nullptr && p.ag_flags == nullptr;
  static const int no_split = getenv("FTB_GEMM_NO_SPLIT") ? atoi(getenv("FTB_GEMM_NO_SPLIT")) : 0;
  const bool split = !PULL && !no_split && p.n_tiles > groups && left > 0 && 2 * left <= groups &&
                     (!push || left <= p.n_tiles / p.tp);
  q.n_full = split ? p.n_tiles - left : p.n_tiles;
  q.n_steps = q.n_full + 2 * (p.n_tiles - q.n_full);
  e = cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_a_own, q);
  return check_cuda(e, "gemm launch");
}

static int gemm_operands_ok(const void* a, const void* b, int m, int n, int k, long long lda, long long ldb) {
  if (m <= 0 || n <= 0 || k <= 0) { set_last_error("gemm: bad sizes m=%d n=%d k=%d", m, n, k); return FTB_ERR_INVALID; }
  if ((n % 8) || (k % 8) || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(a) & 15) ||
      (reinterpret_cast<uintptr_t>(b) & 15)) {
    set_last_error("gemm: n, k and the leading dimensions must be multiples of 8 and pointers 16-byte aligned");
    return FTB_ERR_INVALID;
  }
  return FTB_OK;
}

// `a_own` (all-gather + GEMM only): the rank's own row shard [rows_own, k], read in place of its rows of `a`.
static int launch_gemm(const void* a, const void* b, int m, int n, int k, long long lda, long long ldb,
                       gemm::Params& p, cudaStream_t st, const void* a_own = nullptr, int rows_own = 0, long long lda_own = 0) {
  const int ok = gemm_operands_ok(a, b, m, n, k, lda, ldb);
  if (ok != FTB_OK) return ok;
  CUtensorMap tm_a, tm_b, tm_a_own;
  if (!make_tmap_2d(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, m, k, lda, gemm::BM, gemm::BK) ||
      !make_tmap_2d(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, n, ldb, gemm::BK, 64)) {
    set_last_error("gemm: cuTensorMapEncodeTiled failed");
    return FTB_ERR_CUDA;
  }
  if (a_own == nullptr) {
    tm_a_own = tm_a;
  } else if (!make_tmap_2d(&tm_a_own, a_own, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_own, k, lda_own, gemm::BM, gemm::BK)) {
    set_last_error("gemm: cuTensorMapEncodeTiled failed (own shard)");
    return FTB_ERR_CUDA;
  }
  p.m = m; p.n = n; p.k = k;
  p.m_blocks = (m + gemm::BM - 1) / gemm::BM;
  p.n_blocks = (n + gemm::BN - 1) / gemm::BN;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // CTA pairs when there are at least two row blocks per owner (and the caller did not opt out).
  static const int force = getenv("FTB_GEMM_NCTA") ? atoi(getenv("FTB_GEMM_NCTA")) : 0;
  int ncta = (p.tp > 1 ? (p.blocks_per_shard % 2 == 0) : (p.m_blocks >= 2)) ? 2 : 1;
  if (force == 1 || force == 2) ncta = (force == 2 && p.tp > 1 && (p.blocks_per_shard % 2)) ? 1 : force;
  const bool pull = p.tp > 1 && p.mc_part != nullptr;
  p.n_tiles = ((p.m_blocks + ncta - 1) / ncta) * p.n_blocks;
  if (ncta == 2) return pull ? launch_variant<2, true>(tm_a, tm_b, tm_a_own, p, sms, st) : launch_variant<2, false>(tm_a, tm_b, tm_a_own, p, sms, st);
  return pull ? launch_variant<1, true>(tm_a, tm_b, tm_a_own, p, sms, st) : launch_variant<1, false>(tm_a, tm_b, tm_a_own, p, sms, st);
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
  return launch_gemm(g->a, g->b, g->m, g->n, g->k, g->lda, g->ldb, p, reinterpret_cast<cudaStream_t>(stream));
}

struct ftb_gemm_rs_ctx {
  int rank, tp, m, n, shard_rows, blocks_per_shard;
  void* recv[gemm::MAX_TP];
  unsigned int* flags[gemm::MAX_TP];
  unsigned int* d_counter;
  unsigned int* d_blk_counter;   // pull mode: arrivals per 128-row block
  void* mc_recv;                 // multicast address of the receive/partial buffers (NULL = push mode)
  unsigned int epoch;
  int form;                      // 0 = not used yet, 1 = fused bf16 calls, 2 = staged calls (bf16 or FP8), 3 = copy-engine calls: the flag words differ
  int staged;                    // bf16 calls: 0 = fused kernel (push or pull), 1 = staged (GEMM per shard group + one reduce)
  long long wait_limit;          // cycles a device-side wait for another rank may last
  // copy-engine exchange
  int copy_engine;               // bf16 calls: the exchange runs on the copy engines beside the GEMM
  int ce_chunks;                 // pieces a row shard leaves in
  void* part;                    // this rank's partial product [m, n] bf16 (local memory)
  unsigned int* d_ready;         // [tp * ce_chunks] "piece of shard d of the partial is complete" (call number)
  unsigned int* d_shard_cnt;     // [tp * ce_chunks]
  unsigned int* d_ce_counter;    // CTA completion counter of the GEMM launches (the reduce kernel has d_counter)
  unsigned int* d_epoch_word;    // the current call number in device memory: source of the four-byte flag copies
  cudaStream_t comm;             // stream of the copies
  cudaEvent_t ev_fork, ev_join;
};

extern "C" FTB_API int ftb_gemm_rs_workspace_bytes(int m, int n, int tp, int64_t* recv_bytes, int64_t* flag_bytes) {
  if (m <= 0 || n <= 0 || tp <= 0 || tp > gemm::MAX_TP || (m % (tp * gemm::BM)) || (n % 64) || !recv_bytes || !flag_bytes) {
    set_last_error("ftb_gemm_rs_workspace_bytes: need 1 <= tp <= 8, m a multiple of tp*128, n a multiple of 64");
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
  c->form = 0;
  c->staged = 0;
  c->wait_limit = kWaitLimitCycles;
  c->copy_engine = 0;
  c->part = nullptr; c->d_ready = nullptr; c->d_shard_cnt = nullptr; c->d_ce_counter = nullptr; c->d_epoch_word = nullptr; c->comm = nullptr; c->ev_fork = nullptr; c->ev_join = nullptr;
  for (int i = 0; i < tp; ++i) {
    if (!recv_ptrs[i] || !flag_ptrs[i]) { delete c; set_last_error("ftb_gemm_rs_ctx_create: null peer pointer"); return FTB_ERR_INVALID; }
    c->recv[i] = recv_ptrs[i];
    c->flags[i] = reinterpret_cast<unsigned int*>(flag_ptrs[i]);
  }
  c->mc_recv = nullptr;
  c->d_counter = nullptr;
  c->d_blk_counter = nullptr;
  const int m_blocks = m / gemm::BM;
  cudaError_t e = cudaMalloc(&c->d_counter, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(c->d_counter, 0, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMalloc(&c->d_blk_counter, sizeof(unsigned int) * m_blocks);
  if (e == cudaSuccess) e = cudaMemset(c->d_blk_counter, 0, sizeof(unsigned int) * m_blocks);
  if (e != cudaSuccess) {
    cudaFree(c->d_counter);        // cudaFree(nullptr) is a no-op
    cudaFree(c->d_blk_counter);
    delete c;
    return check_cuda(e, "ftb_gemm_rs_ctx_create");
  }
  *out = c;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs_ctx_set_multicast(ftb_gemm_rs_ctx* c, void* mc_recv_ptr) {
  if (!c) { set_last_error("ftb_gemm_rs_ctx_set_multicast: null context"); return FTB_ERR_INVALID; }
  if (c->epoch != 0) { set_last_error("ftb_gemm_rs_ctx_set_multicast: must be called before the first ftb_gemm_rs"); return FTB_ERR_INVALID; }
  c->mc_recv = mc_recv_ptr;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs_ctx_set_wait_limit(ftb_gemm_rs_ctx* c, int64_t cycles) {
  if (!c || cycles <= 0) { set_last_error("ftb_gemm_rs_ctx_set_wait_limit: need a context and a positive cycle count"); return FTB_ERR_INVALID; }
  c->wait_limit = cycles;
  return FTB_OK;
}

extern "C" FTB_API int ftb_gemm_rs_ctx_destroy(ftb_gemm_rs_ctx* c) {
  if (!c) return FTB_OK;
  cudaFree(c->d_counter);
  cudaFree(c->d_blk_counter);
  cudaFree(c->part);
  cudaFree(c->d_ready);
  cudaFree(c->d_shard_cnt);
  cudaFree(c->d_ce_counter);
  cudaFree(c->d_epoch_word);
  if (c->comm) cudaStreamDestroy(c->comm);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  delete c;
  return FTB_OK;
}

// ---------------------------------------------------------------------------------------------
// Block-scaled FP8 GEMM + reduce-scatter (the FP8 shape family of the tensor-parallel path).
//
// Two phases per call, all kernels of this library: (1) the block-scaled FP8 GEMM writes this rank's whole
// partial product [m, n] as bf16 into its own peer-mapped buffer and a one-warp kernel publishes "partial
// e is complete" in every peer's flag words; (2) the reduce kernel waits (bounded) for the same word from
// every peer and writes this rank's row shard as the sum over ranks: with an NVSwitch multicast mapping one
// multimem.ld_reduce per 16 bytes (the switch adds the eight partials), else plain peer loads added in
// fp32 in rank order.  When its last CTA is through, it tells every peer that their buffers have been read,
// which is what the next call waits for before the GEMM overwrites the partial.  The exchange is not
// overlapped with the GEMM yet (the reduce starts when every rank has finished its product).
// Flag words of rank d in this form: [src] = last complete partial of rank src, [tp + src] = last call in
// which rank src finished reading rank d's partial.  Every kernel here waits on other GPUs only.
namespace ftb {
namespace gemm {

__global__ void rs_fp8_wait_kernel(const unsigned int* flags, int first, int tp, unsigned int target, int* status, long long wait_limit) {
  const int i = threadIdx.x;
  if (i >= tp) return;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
  const long long t0 = clock64();
  while (ld_acquire_sys(flags + first + i) < target) {
    if (clock64() - t0 > wait_limit) {
      if (status != nullptr) atomicCAS(status, 0, FTB_ERR_TIMEOUT);
      return;
    }
  }
}

struct RsFp8Ptrs {
  unsigned int* flags[MAX_TP];
  const __nv_bfloat16* recv[MAX_TP];
};

// ranks d0 .. d0 + nd - 1 learn that this rank's partial of their rows is complete
__global__ void rs_fp8_publish_kernel(RsFp8Ptrs q, int d0, int nd, int word, unsigned int value, const int* status) {
  const int d = d0 + static_cast<int>(threadIdx.x);
  if (static_cast<int>(threadIdx.x) >= nd) return;
  // after a timeout the partial of this call may be incomplete: the peers must not be told otherwise
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  __threadfence_system();
  st_release_sys(q.flags[d] + word, value);
}

__global__ void __launch_bounds__(256, 3) rs_fp8_reduce_kernel(RsFp8Ptrs q, const __nv_bfloat16* mc_part, __nv_bfloat16* out,
                                                           long long ldo, int shard_rows, int n, int rank, int tp,
                                                           unsigned int epoch, unsigned int* counter, int* status, long long wait_limit) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
  __syncthreads();
  if (threadIdx.x < tp && !s_abort) {
    // partial `epoch` of every rank is complete
    const long long t0 = clock64();
    while (ld_acquire_sys(q.flags[rank] + threadIdx.x) < epoch) {
      if (clock64() - t0 > wait_limit) {
        s_abort = 1;
        if (status != nullptr) atomicCAS(status, 0, FTB_ERR_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  if (!s_abort) {
    const int vec_per_row = n / 8;
    const long long total = static_cast<long long>(shard_rows) * vec_per_row;
    const long long row0 = static_cast<long long>(rank) * shard_rows;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    constexpr int kU = 4;   // loads in flight per thread (one at a time moved 250 GB/s); three CTAs per SM
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * kU) {
      uint4 o[kU];
      long long off[kU], dst[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const long long i = i0 + u * stride;
        const long long r = i < total ? i / vec_per_row : 0;
        const int c8 = i < total ? static_cast<int>(i - r * vec_per_row) : 0;
        off[u] = (row0 + r) * n + c8 * 8;
        dst[u] = r * ldo + c8 * 8;
      }
      if (mc_part != nullptr) {
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (i0 + u * stride < total) o[u] = multimem_ld_reduce_bf16x8(mc_part + off[u]);
      } else {
        float acc[kU][8];
#pragma unroll
        for (int u = 0; u < kU; ++u)
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
        for (int src = 0; src < tp; ++src) {
          uint4 v[kU];
#pragma unroll
          for (int u = 0; u < kU; ++u)
            v[u] = (i0 + u * stride < total) ? *reinterpret_cast<const uint4*>(q.recv[src] + off[u]) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              acc[u][2 * k] += __uint_as_float(w[k] << 16);
              acc[u][2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          o[u].x = pack_bf16x2(acc[u][0], acc[u][1]); o[u].y = pack_bf16x2(acc[u][2], acc[u][3]);
          o[u].z = pack_bf16x2(acc[u][4], acc[u][5]); o[u].w = pack_bf16x2(acc[u][6], acc[u][7]);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (i0 + u * stride < total) *reinterpret_cast<uint4*>(out + dst[u]) = o[u];
    }
  }
  // the last CTA tells every peer that this rank has read their partials of this call
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) == gridDim.x - 1u) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *counter = 0u;
    if (threadIdx.x < tp) st_release_sys(q.flags[threadIdx.x] + tp + rank, epoch);
  }
}



}  // namespace gemm
}  // namespace ftb

// Staged driver shared by the bf16 and FP8 forms.  The GEMM runs once per group of row shards, the groups in
// rotated order (the group after this rank's own first, its own last), each launch writing rows of this rank's
// partial [m, n] in its peer-mapped buffer; after a group the owners of its shards learn that this rank's
// partial of their rows is complete.  When the own group is done only the stragglers and one pass over this
// rank's shard are left: the reduce kernel.  `gemm_rows(row0, rows, c)` launches the GEMM of rows
// [row0, row0 + rows) into c (row stride n).
template <typename GemmRows>
static int staged_gemm_rs(ftb_gemm_rs_ctx* c, GemmRows gemm_rows, void* out, int64_t ldo, int32_t* status, cudaStream_t st) {
  using namespace ftb;
  c->epoch += 1;
  gemm::RsFp8Ptrs q;
  memset(&q, 0, sizeof(q));
  for (int i = 0; i < c->tp; ++i) {
    q.flags[i] = c->flags[i];
    q.recv[i] = reinterpret_cast<const __nv_bfloat16*>(c->recv[i]);
  }
  // every peer has read the partial of the call before (their words start at [tp])
  gemm::rs_fp8_wait_kernel<<<1, 32, 0, st>>>(c->flags[c->rank], c->tp, c->tp, c->epoch - 1u, status, c->wait_limit);
  int rc = check_cuda(cudaGetLastError(), "rs wait launch");
  if (rc != FTB_OK) return rc;
  // Shards per GEMM launch.  Nothing overlaps the exchange in this protocol (a rank's own group comes last, so
  // no reduce can start before the last launch), and every extra launch costs a partial wave of tiles: at the
  // cfg4 shape on 8 GPUs one launch took 0.411 ms, two 0.431, four 0.483.  So: one group.  The loop below
  // stays general for the day the reduce of a finished group runs beside the next launch.
  int g = c->tp;
  const int n_groups = c->tp / g;
  const int own = c->rank / g;
  __nv_bfloat16* part = reinterpret_cast<__nv_bfloat16*>(c->recv[c->rank]);
  for (int s = 1; s <= n_groups; ++s) {
    const int gi = (own + s) % n_groups;
    const long long row0 = static_cast<long long>(gi) * g * c->shard_rows;
    rc = gemm_rows(row0, g * c->shard_rows, part + row0 * c->n);
    if (rc != FTB_OK) return rc;
    gemm::rs_fp8_publish_kernel<<<1, 32, 0, st>>>(q, gi * g, g, c->rank, c->epoch, status);
    rc = check_cuda(cudaGetLastError(), "rs publish launch");
    if (rc != FTB_OK) return rc;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  gemm::rs_fp8_reduce_kernel<<<sms * 3, 256, 0, st>>>(q, reinterpret_cast<const __nv_bfloat16*>(c->mc_recv),
                                                      reinterpret_cast<__nv_bfloat16*>(out), ldo, c->shard_rows, c->n, c->rank,
                                                      c->tp, c->epoch, c->d_counter, status, c->wait_limit);
  return check_cuda(cudaGetLastError(), "rs reduce launch");
}

// Copy-engine exchange.  One persistent GEMM launch in the push protocol's tile order (the other ranks' row shards
// first, rotated by rank, the own shard last).  Tiles of other ranks' rows are stored into this rank's local partial
// [m, n]; a shard leaves in `chunks` pieces of consecutive row blocks: when the last tile of a piece is stored its
// word in ready[] takes the call number, a second stream waits for that word with a stream memory operation (and,
// before the first piece, until the owner has read the previous call's pieces), copies the piece into the owner's
// receive slot with an ordinary device-to-device copy, which the copy engines carry out, and raises the owner's
// flag for (source, piece) with a four-byte copy of the call number.  The epilogue of the own rows waits (bounded)
// for the peers' flags of the piece and adds their partials to the accumulator in fp32: the sum is written once,
// there is no reduce pass, and no SM moves exchange data.  The second stream runs no kernel (a kernel there might
// find every SM held by GEMM CTAs that wait for it) and its waits have no time limit: a rank that never arrives
// stalls it.  A launch that finds the status word set, or whose waits ran out, raises every ready word so that the
// waits of the second stream end whatever became of the GEMM.
static int copy_engine_gemm_rs(ftb_gemm_rs_ctx* c, const void* a, const void* b, void* out, int k_local, int64_t lda,
                               int64_t ldb, int64_t ldo, int32_t* status, cudaStream_t st) {
  using namespace ftb;
  if (c->form == 1 || c->form == 2) { set_last_error("ftb_gemm_rs: this context has served calls of another protocol (the flag words differ)"); return FTB_ERR_INVALID; }
  static StreamValue32Fn wait32 = get_stream_memop("cuStreamWaitValue32");
  static StreamValue32Fn write32 = get_stream_memop("cuStreamWriteValue32");
  if (!wait32 || !write32) { set_last_error("ftb_gemm_rs: stream memory operations are not available"); return FTB_ERR_UNSUPPORTED; }
  c->form = 3;
  c->epoch += 1;
  const unsigned int epoch = c->epoch;
  const int tp = c->tp, rank = c->rank;
  const int chunks = c->ce_chunks;
  const long long slot = static_cast<long long>(c->shard_rows) * c->n;       // elements of one row shard
  // row groups as the CTA groups take them (pairs of row blocks when the shard has an even number of them); group g
  // belongs to piece floor(g * chunks / groups), so piece p starts at group ceil(p * groups / chunks)
  const int rows_per_group = (c->blocks_per_shard % 2 == 0 ? 2 : 1) * gemm::BM;
  const int groups = c->shard_rows / rows_per_group;
  auto piece_row0 = [&](int pc) { return ((pc * groups + chunks - 1) / chunks) * rows_per_group; };
  __nv_bfloat16* part = reinterpret_cast<__nv_bfloat16*>(c->part);
  cudaError_t e = cudaEventRecord(c->ev_fork, st);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(c->comm, c->ev_fork, 0);
  if (e != cudaSuccess) return check_cuda(e, "gemm_rs copy-engine fork");
  gemm::Params p;
  memset(&p, 0, sizeof(p));
  p.tp = tp; p.rank = rank; p.shard_rows = c->shard_rows; p.blocks_per_shard = c->blocks_per_shard;
  p.epoch = epoch;
  p.c = part; p.ldc = c->n;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.status = status;
  p.wait_limit = c->wait_limit;
  p.ce_ready = c->d_ready;
  p.ce_cnt = c->d_shard_cnt;
  p.ce_chunks = chunks;
  p.ce_groups = groups;
  p.ce_group_blocks = rows_per_group / gemm::BM;
  p.counter = c->d_ce_counter;
  for (int i = 0; i < tp; ++i) {
    p.flags[i] = c->flags[i];
    p.recv[i] = reinterpret_cast<__nv_bfloat16*>(c->recv[i]);
  }
  const int n_blocks = (c->n + gemm::BN - 1) / gemm::BN;
  // 4 epilogue warps per tile and row block, a whole tile counts 2
  for (int pc = 0; pc < chunks; ++pc)
    p.ce_target[pc] = epoch * static_cast<unsigned int>((piece_row0(pc + 1) - piece_row0(pc)) / gemm::BM) * static_cast<unsigned int>(n_blocks) * 8u;
  int rc = launch_gemm(a, b, c->m, c->n, k_local, lda, ldb, p, st);
  if (rc != FTB_OK) return rc;
  // ---- exchange on the second stream, piece after piece in the order in which they complete.  (One stream per
  // destination and flags raised by stream writes to the peer were measured too: no faster; the copy engines give
  // a rank about 500 GB/s in copies of this size whatever the number of streams.)
  CUresult r = write32(reinterpret_cast<CUstream>(c->comm), reinterpret_cast<CUdeviceptr>(c->d_epoch_word), epoch, CU_STREAM_WRITE_VALUE_DEFAULT);
  if (r != CUDA_SUCCESS) { set_last_error("ftb_gemm_rs: cuStreamWriteValue32 failed (%d)", static_cast<int>(r)); return FTB_ERR_CUDA; }
  for (int s = 1; s < tp; ++s) {
    const int d = (rank + s) % tp;
    for (int ch = 0; ch < chunks; ++ch) {
      r = wait32(reinterpret_cast<CUstream>(c->comm), reinterpret_cast<CUdeviceptr>(c->d_ready + d * chunks + ch), epoch, CU_STREAM_WAIT_VALUE_GEQ);
      // rank d has read the pieces of the call before (its word [tp * chunks + d] in this rank's flags)
      if (r == CUDA_SUCCESS && ch == 0 && epoch > 1u)
        r = wait32(reinterpret_cast<CUstream>(c->comm), reinterpret_cast<CUdeviceptr>(c->flags[rank] + tp * chunks + d), epoch - 1u, CU_STREAM_WAIT_VALUE_GEQ);
      if (r != CUDA_SUCCESS) { set_last_error("ftb_gemm_rs: cuStreamWaitValue32 failed (%d)", static_cast<int>(r)); return FTB_ERR_CUDA; }
      const long long off = static_cast<long long>(piece_row0(ch)) * c->n;
      const size_t bytes = static_cast<size_t>(piece_row0(ch + 1) - piece_row0(ch)) * c->n * 2;
      e = cudaMemcpyAsync(reinterpret_cast<__nv_bfloat16*>(c->recv[d]) + rank * slot + off, part + d * slot + off, bytes,
                          cudaMemcpyDeviceToDevice, c->comm);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(c->flags[d] + rank * chunks + ch, c->d_epoch_word, sizeof(unsigned int), cudaMemcpyDeviceToDevice, c->comm);
      if (e != cudaSuccess) return check_cuda(e, "gemm_rs copy-engine copy");
    }
  }
  e = cudaEventRecord(c->ev_join, c->comm);
  if (e != cudaSuccess) return check_cuda(e, "gemm_rs copy-engine join");
  // the next call's GEMM overwrites the partial: not before this call's copies have read it
  return check_cuda(cudaStreamWaitEvent(st, c->ev_join, 0), "gemm_rs copy-engine join wait");
}

extern "C" FTB_API int ftb_gemm_rs(ftb_gemm_rs_ctx* c, const void* a, const void* b, void* out, int k_local,
                                   int64_t lda, int64_t ldb, int64_t ldo, int32_t* status, void* stream) {
  if (!c || !a || !b || !out) { set_last_error("ftb_gemm_rs: null pointer"); return FTB_ERR_INVALID; }
  if ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) { set_last_error("ftb_gemm_rs: out alignment"); return FTB_ERR_INVALID; }
  // a rejected call must leave the call counter alone: the peers' flag targets are derived from it
  const int ok = gemm_operands_ok(a, b, c->m, c->n, k_local, lda, ldb);
  if (ok != FTB_OK) return ok;
  if (c->copy_engine) return copy_engine_gemm_rs(c, a, b, out, k_local, lda, ldb, ldo, status, reinterpret_cast<cudaStream_t>(stream));
  if (c->staged) {
    if (c->form == 1 || c->form == 3) { set_last_error("ftb_gemm_rs: this context has served calls of another protocol (the flag words differ)"); return FTB_ERR_INVALID; }
    c->form = 2;
    const int n = c->n;
    auto rows = [&](long long row0, int m_rows, __nv_bfloat16* dst) -> int {
      ftb_gemm_args g;
      memset(&g, 0, sizeof(g));
      g.a = static_cast<const __nv_bfloat16*>(a) + row0 * lda;
      g.b = b;
      g.c = dst;
      g.m = m_rows; g.n = n; g.k = k_local;
      g.lda = lda; g.ldb = ldb; g.ldc = n;
      g.status = status;
      return ftb_gemm_bf16(&g, stream);
    };
    return staged_gemm_rs(c, rows, out, ldo, status, reinterpret_cast<cudaStream_t>(stream));
  }
  if (c->form == 2 || c->form == 3) { set_last_error("ftb_gemm_rs: this context serves calls of another protocol (the flag words differ)"); return FTB_ERR_INVALID; }
  c->form = 1;
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
  p.mc_part = reinterpret_cast<const __nv_bfloat16*>(c->mc_recv);
  p.blk_counter = c->d_blk_counter;
  p.wait_limit = c->wait_limit;
  return launch_gemm(a, b, c->m, c->n, k_local, lda, ldb, p, st);
}

extern "C" FTB_API int ftb_gemm_rs_fp8(ftb_gemm_rs_ctx* c, const void* a, const void* b, const float* a_scale,
                                       const float* b_scale, void* out, int k_local, int64_t lda, int64_t ldb,
                                       int64_t a_scale_ld, int64_t b_scale_ld, int64_t ldo, int32_t* status, void* stream) {
  if (!c || !a || !b || !a_scale || !b_scale || !out) { set_last_error("ftb_gemm_rs_fp8: null pointer"); return FTB_ERR_INVALID; }
  if ((ldo % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) { set_last_error("ftb_gemm_rs_fp8: out alignment"); return FTB_ERR_INVALID; }
  if (c->form == 1 || c->form == 3) { set_last_error("ftb_gemm_rs_fp8: this context serves bf16 calls of another protocol (the flag words differ)"); return FTB_ERR_INVALID; }
  if ((c->n % 128) || (k_local % 128)) { set_last_error("ftb_gemm_rs_fp8: n and k_local must be multiples of 128"); return FTB_ERR_INVALID; }
  if (k_local <= 0 || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) {
    set_last_error("ftb_gemm_rs_fp8: operands must be 16-byte aligned with leading dimensions that are multiples of 16");
    return FTB_ERR_INVALID;
  }
  c->form = 2;
  const int n = c->n;
  auto rows = [&](long long row0, int m_rows, __nv_bfloat16* dst) -> int {
    ftb_gemm_fp8_args g;
    memset(&g, 0, sizeof(g));
    g.a = static_cast<const uint8_t*>(a) + row0 * lda;
    g.b = b;
    g.c = dst;
    g.a_scale = a_scale + row0 * a_scale_ld;
    g.b_scale = b_scale;
    g.m = m_rows; g.n = n; g.k = k_local;
    g.lda = lda; g.ldb = ldb; g.ldc = n;
    g.a_scale_ld = a_scale_ld; g.b_scale_ld = b_scale_ld;
    g.status = status;
    return ftb_gemm_fp8_blockscaled(&g, stream);
  };
  return staged_gemm_rs(c, rows, out, ldo, status, reinterpret_cast<cudaStream_t>(stream));
}

// bf16 calls of this context exchange their partials on the copy engines (1) or inside the GEMM kernel (0).  Must be
// chosen before the first call.  Allocates the local partial [m, n] and the second stream.
extern "C" FTB_API int ftb_gemm_rs_ctx_set_copy_engine(ftb_gemm_rs_ctx* c, int on) {
  if (!c) { set_last_error("ftb_gemm_rs_ctx_set_copy_engine: null context"); return FTB_ERR_INVALID; }
  if (c->epoch != 0) { set_last_error("ftb_gemm_rs_ctx_set_copy_engine: must be called before the first call"); return FTB_ERR_INVALID; }
  if (on && c->part == nullptr) {
    cudaError_t e = cudaMalloc(&c->part, static_cast<size_t>(c->m) * c->n * 2);
    // A shard leaves in up to four pieces (whole CTA-pair row groups each), as long as the second stream has at
    // most eight copies per call to issue: the pieces of the shard computed last arrive while the own rows are
    // still being multiplied.
    const int groups = c->blocks_per_shard % 2 == 0 ? c->blocks_per_shard / 2 : c->blocks_per_shard;
    // measured: tp = 2: 4 pieces (2: +12 %, 3 and 6: +5 %); tp = 4: 2 pieces (1 and 4: +7 %)
    int chunks = c->tp == 2 ? 4 : c->tp <= 4 ? 2 : 1;
    if (const char* ev = getenv("FTB_RS_PIECES")) chunks = atoi(ev);      // tuning override
    if (chunks > 8) chunks = 8;
    if (chunks > groups) chunks = groups;
    if (chunks < 1) chunks = 1;
    c->ce_chunks = chunks;
    const size_t words = sizeof(unsigned int) * gemm::MAX_TP * 8;
    if (e == cudaSuccess) e = cudaMalloc(&c->d_ready, words);
    if (e == cudaSuccess) e = cudaMemset(c->d_ready, 0, words);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_shard_cnt, words);
    if (e == cudaSuccess) e = cudaMemset(c->d_shard_cnt, 0, words);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_epoch_word, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&c->d_ce_counter, sizeof(unsigned int));

    if (e == cudaSuccess) e = cudaMemset(c->d_ce_counter, 0, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->comm, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming);
    if (e != cudaSuccess) return check_cuda(e, "ftb_gemm_rs_ctx_set_copy_engine");
  }
  c->copy_engine = on ? 1 : 0;
  return FTB_OK;
}

// bf16 calls of this context use the staged protocol (1) or the fused kernel (0, the default).  Must be chosen
// before the first call: the two use the flag words differently.
extern "C" FTB_API int ftb_gemm_rs_ctx_set_staged(ftb_gemm_rs_ctx* c, int staged) {
  if (!c) { set_last_error("ftb_gemm_rs_ctx_set_staged: null context"); return FTB_ERR_INVALID; }
  if (c->epoch != 0) { set_last_error("ftb_gemm_rs_ctx_set_staged: must be called before the first call"); return FTB_ERR_INVALID; }
  c->staged = staged ? 1 : 0;
  return FTB_OK;
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



// ---------------------------------------------------------------------------------------------
// All-gather + GEMM (the column-parallel sibling that feeds the row-parallel GEMM + reduce-scatter).
//
// Rank r holds the row shard A_r [m / tp, k] and its weight columns B_r [k, n_local]; every rank computes
// C_r = A . B_r with A [m, k] the shards of all ranks stacked in rank order.  The shards travel on the copy
// engines: a second stream copies this rank's shard into every peer's gather buffer (rank + 1 first) and raises
// the peer's flag with a four-byte copy of the call number; it runs no kernel.  One persistent GEMM launch reads
// A from the rank's gather buffer, own rows first, then the shards in the order in which they are sent to it; its
// TMA producer waits (bounded) for a shard's flag before it loads the shard's first tile.  The kernel's last CTA
// tells the peers that the gather buffer has been read, which is what their next call's copies wait for.
// Flag words of rank d: [src] = last call whose shard from rank src has landed, [tp + src] = last call in which
// rank src finished reading rank d's shard out of src's own gather buffer.
struct ftb_ag_gemm_ctx {
  int rank, tp, m, k, shard_rows;
  void* ag[gemm::MAX_TP];              // gather buffers [m, k] bf16 (peer-mapped)
  unsigned int* flags[gemm::MAX_TP];
  unsigned int* d_counter;
  unsigned int* d_epoch_word;
  cudaStream_t comm;
  cudaEvent_t ev_fork, ev_join;
  unsigned int epoch;
  long long wait_limit;
};

extern "C" FTB_API int ftb_ag_gemm_workspace_bytes(int m, int k, int tp, int64_t* ag_bytes, int64_t* flag_bytes) {
  if (m <= 0 || k <= 0 || tp <= 0 || tp > gemm::MAX_TP || (m % (tp * gemm::BM)) || (k % 8) || !ag_bytes || !flag_bytes) {
    set_last_error("ftb_ag_gemm_workspace_bytes: need 1 <= tp <= 8, m a multiple of tp*128, k a multiple of 8");
    return FTB_ERR_INVALID;
  }
  *ag_bytes = static_cast<int64_t>(m) * k * 2;
  *flag_bytes = 256;
  return FTB_OK;
}

extern "C" FTB_API int ftb_ag_gemm_ctx_create(ftb_ag_gemm_ctx** out, int rank, int tp, int m, int k, void* const* ag_ptrs,
                                              void* const* flag_ptrs) {
  int64_t ab, fb;
  if (!out || !ag_ptrs || !flag_ptrs || rank < 0 || rank >= tp) { set_last_error("ftb_ag_gemm_ctx_create: bad argument"); return FTB_ERR_INVALID; }
  int rc = ftb_ag_gemm_workspace_bytes(m, k, tp, &ab, &fb);
  if (rc != FTB_OK) return rc;
  ftb_ag_gemm_ctx* c = new ftb_ag_gemm_ctx();
  memset(c, 0, sizeof(*c));
  c->rank = rank; c->tp = tp; c->m = m; c->k = k; c->shard_rows = m / tp;
  c->wait_limit = kWaitLimitCycles;
  for (int i = 0; i < tp; ++i) {
    if (!ag_ptrs[i] || !flag_ptrs[i]) { delete c; set_last_error("ftb_ag_gemm_ctx_create: null peer pointer"); return FTB_ERR_INVALID; }
    c->ag[i] = ag_ptrs[i];
    c->flags[i] = reinterpret_cast<unsigned int*>(flag_ptrs[i]);
  }
  cudaError_t e = cudaMalloc(&c->d_counter, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(c->d_counter, 0, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMalloc(&c->d_epoch_word, sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->comm, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming);
  if (e != cudaSuccess) { ftb_ag_gemm_ctx_destroy(c); return check_cuda(e, "ftb_ag_gemm_ctx_create"); }
  *out = c;
  return FTB_OK;
}

extern "C" FTB_API int ftb_ag_gemm_ctx_set_wait_limit(ftb_ag_gemm_ctx* c, int64_t cycles) {
  if (!c || cycles <= 0) { set_last_error("ftb_ag_gemm_ctx_set_wait_limit: need a context and a positive cycle count"); return FTB_ERR_INVALID; }
  c->wait_limit = cycles;
  return FTB_OK;
}

extern "C" FTB_API int ftb_ag_gemm_ctx_destroy(ftb_ag_gemm_ctx* c) {
  if (!c) return FTB_OK;
  cudaFree(c->d_counter);
  cudaFree(c->d_epoch_word);
  if (c->comm) cudaStreamDestroy(c->comm);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  delete c;
  return FTB_OK;
}

extern "C" FTB_API int ftb_ag_gemm(ftb_ag_gemm_ctx* c, const void* a_shard, const void* b, void* out, int n_local, int64_t lda,
                                   int64_t ldb, int64_t ldc, int32_t* status, void* stream) {
  if (!c || !a_shard || !b || !out) { set_last_error("ftb_ag_gemm: null pointer"); return FTB_ERR_INVALID; }
  if ((ldc % 8) || (reinterpret_cast<uintptr_t>(out) & 15) || (lda % 8) || (reinterpret_cast<uintptr_t>(a_shard) & 15)) {
    set_last_error("ftb_ag_gemm: a_shard and out must be 16-byte aligned with leading dimensions that are multiples of 8");
    return FTB_ERR_INVALID;
  }
  const int ok = gemm_operands_ok(c->ag[c->rank], b, c->m, n_local, c->k, c->k, ldb);
  if (ok != FTB_OK) return ok;
  static StreamValue32Fn wait32 = get_stream_memop("cuStreamWaitValue32");
  static StreamValue32Fn write32 = get_stream_memop("cuStreamWriteValue32");
  if (!wait32 || !write32) { set_last_error("ftb_ag_gemm: stream memory operations are not available"); return FTB_ERR_UNSUPPORTED; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  c->epoch += 1;
  const unsigned int epoch = c->epoch;
  const int tp = c->tp, rank = c->rank;
  const size_t shard_bytes = static_cast<size_t>(c->shard_rows) * c->k * 2;
  cudaError_t e = cudaEventRecord(c->ev_fork, st);      // the shard is ready on the caller's stream
  if (e == cudaSuccess) e = cudaStreamWaitEvent(c->comm, c->ev_fork, 0);
  if (e != cudaSuccess) return check_cuda(e, "ag_gemm fork");
  // ---- second stream: the shard goes to the peers, rank + 1 first (the own rows are read where they lie)
  CUresult r = write32(reinterpret_cast<CUstream>(c->comm), reinterpret_cast<CUdeviceptr>(c->d_epoch_word), epoch, CU_STREAM_WRITE_VALUE_DEFAULT);
  if (r != CUDA_SUCCESS) { set_last_error("ftb_ag_gemm: cuStreamWriteValue32 failed (%d)", static_cast<int>(r)); return FTB_ERR_CUDA; }
  for (int s = 1; s < tp; ++s) {
    const int d = (rank + s) % tp;
    // rank d has read the gather buffer of the call before (its word [tp + d] in this rank's flags)
    if (epoch > 1u) {
      r = wait32(reinterpret_cast<CUstream>(c->comm), reinterpret_cast<CUdeviceptr>(c->flags[rank] + tp + d), epoch - 1u, CU_STREAM_WAIT_VALUE_GEQ);
      if (r != CUDA_SUCCESS) { set_last_error("ftb_ag_gemm: cuStreamWaitValue32 failed (%d)", static_cast<int>(r)); return FTB_ERR_CUDA; }
    }
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c->ag[d]) + static_cast<size_t>(rank) * c->shard_rows * c->k;
    // A contiguous shard goes as one linear copy, which the copy engines carry out.  (A pitched copy may be run
    // by a kernel of the driver's; on a GPU whose SMs are held by GEMM CTAs that wait for this very copy such a
    // kernel has no place to run until the waits give up.)
    if (lda == c->k)
      e = cudaMemcpyAsync(dst, a_shard, shard_bytes, cudaMemcpyDeviceToDevice, c->comm);
    else
      e = cudaMemcpy2DAsync(dst, static_cast<size_t>(c->k) * 2, a_shard, static_cast<size_t>(lda) * 2, static_cast<size_t>(c->k) * 2,
                            static_cast<size_t>(c->shard_rows), cudaMemcpyDeviceToDevice, c->comm);
    if (e == cudaSuccess) e = cudaMemcpyAsync(c->flags[d] + rank, c->d_epoch_word, sizeof(unsigned int), cudaMemcpyDeviceToDevice, c->comm);
    if (e != cudaSuccess) return check_cuda(e, "ag_gemm copy");
  }
  e = cudaEventRecord(c->ev_join, c->comm);
  if (e != cudaSuccess) return check_cuda(e, "ag_gemm join");
  // ---- the GEMM over the gather buffer
  gemm::Params p;
  memset(&p, 0, sizeof(p));
  p.tp = tp; p.rank = rank; p.shard_rows = c->shard_rows; p.blocks_per_shard = c->shard_rows / gemm::BM;
  p.epoch = epoch;
  p.c = reinterpret_cast<__nv_bfloat16*>(out); p.ldc = ldc;
  p.status = status;
  p.wait_limit = c->wait_limit;
  p.ag_flags = c->flags[rank];
  p.counter = c->d_counter;
  for (int i = 0; i < tp; ++i) p.flags[i] = c->flags[i];
  int rc = launch_gemm(c->ag[rank], b, c->m, n_local, c->k, c->k, ldb, p, st, a_shard, c->shard_rows, lda);
  if (rc != FTB_OK) return rc;
  // the caller may overwrite its shard once the copies have read it
  return check_cuda(cudaStreamWaitEvent(st, c->ev_join, 0), "ag_gemm join wait");
}
