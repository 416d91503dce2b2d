// Top-k sparse MLA forward, role-split CTA pair with Q held in tensor memory (bf16 KV).
//
// Same division of labour as sparse_mla_duo.cu (CTA 0: S = Q.K^T + softmax, CTA 1: O += P.V, P sent over
// distributed shared memory) with one change that matters for the K ring: Q [128 heads x 576] is not kept
// in shared memory (147 KB) but in CTA 0's tensor memory (288 of 512 columns, two bf16 per 32-bit column)
// and enters the MMA as the TMEM A operand.  That frees the shared memory for a 9-slot ring of K column
// blocks (a whole tile in flight instead of 4 blocks: the refill latency of a slot, about 3000 cycles from
// the commit that frees it to the landing of the new rows, no longer paces the MMAs) and for two local
// staging buffers of P.  The softmax writes P into local shared memory (conflict-free 16-byte stores) and
// each warp then sends its 4 KB with one bulk copy over distributed shared memory that completes on the
// P barrier of CTA 1; 16-byte st.shared::cluster stores scattered over 32 rows per instruction took about
// 6000 cycles per tile.  TMEM of CTA 0: Q in columns 0-287, one S buffer [128 x 128] in columns 320-447
// (the softmax copies S to registers at once, so one buffer is enough).  Q arrives by nine TMA tile loads;
// the epilogue of CTA 1 runs on eight warps, stages O in shared memory in the swizzled tile layout and
// leaves through eight TMA tile stores (256 bulk stores of half rows took 6000 cycles to issue).
//
// KV rows are fetched with TMA tile::gather4 (four row indices per instruction, boxes of 64 columns x 1 row,
// 128B swizzle, never multicast), one producer warp per 64-column block and every lane issuing its own
// gathers: one warp alone issues a gather every 67 cycles, nine warps together one every 12.  The copies
// are writes of the async proxy, like the reads of the MMA, so the MMA issuer needs no proxy fence: with
// cp.async producers that fence cost the issuer about 1300 cycles per pair of blocks while copies were in
// flight, and the tensor pipe ran dry behind it.
//
// Warps (576 threads per CTA): CTA 0: 0-7 softmax (two threads per head row), 8 MMA issuer, 9-17 K producers.
// CTA 1: 0-3 correction, 4 relay, 0-7 epilogue, 8 MMA issuer, 9-16 V producers.  Every wait is bounded.
#include "sm100.cuh"
#include "tmap.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace mla4 {

constexpr int kDqk = 576;
constexpr int kNChunk = 9;
constexpr int kNT = 128;                       // gathered rows per tile
constexpr int kQBlock = 128 * 128;             // 16384: [128 heads x 128 B]
constexpr int kNK = 9;                         // K ring slots (Q lives in TMEM): one whole tile
constexpr int kKSlot = kNT * 128;              // 16384: [128 rows x 128 B]
constexpr int kNV = 4;                         // V ring slots
constexpr int kVSlabRows = 32;
constexpr int kVBlock = kVSlabRows * 128;      // 4096: one 64-column block of a slab
constexpr int kVSlab = 8 * kVBlock;            // 32768
constexpr int kPBuf = 2 * kQBlock;             // 32768: P [128 heads x 128 rows] bf16 as two 64-row blocks
// CTA 0 layout: K ring | P staging x 2 | misc (Q is staged in ring slots 0-8 once, then moved to TMEM).
// CTA 1 layout: V ring | P x 2 | misc; after the last tile the V ring stages O as eight 64-column blocks.
constexpr int kOff0K = 0;
constexpr int kOff0P = kOff0K + kNK * kKSlot;              // 147456
constexpr int kOff0Misc = kOff0P + 2 * kPBuf;              // 212992
constexpr int kOff1P = kNV * kVSlab;                       // 131072
constexpr int kOff1Misc = kOff1P + 2 * kPBuf;              // 196608
constexpr int kSmemBytes = kOff0Misc + 4096 + 1024;        // the larger of the two + misc + alignment slack
constexpr int kThreads = 576;
constexpr uint32_t kColQ = 0;                  // TMEM columns of CTA 0: Q (288), then S
constexpr uint32_t kColS = 320;

struct Params {
  const __nv_bfloat16* q;
  const __nv_bfloat16* kv;
  const int32_t* indices;
  __nv_bfloat16* out;
  float* lse;
  int s_q, h, s_kv, topk;
  long long q_st, q_sh, kv_sr, idx_st, out_st, out_sh, lse_st;
  float scale_log2;
  int lse_base2;
  int* status;
};

struct Misc0 {   // CTA 0
  unsigned long long k_full[kNK];   // one arrival announcing 16 KB of gathers
  unsigned long long k_free[kNK];   // tcgen05.commit
  unsigned long long s_full[2];     // tcgen05.commit (index 0 used: one S buffer)
  unsigned long long s_free[2];     // 8 softmax warps (index 0 used)
  unsigned long long p_free[2];     // relay warp of CTA 1 (remote arrival)
  unsigned long long q_full;        // one arrival announcing the 9 tile loads of Q
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int bad_index;
  uint32_t valid_mask[4][4];        // per tile (mod 4): 128 validity bits
  float xchg[2][256];               // row maximum / row sum exchange between the two threads of a head row
};
struct Misc1 {   // CTA 1
  unsigned long long v_full[kNV];   // one arrival announcing 32 KB of gathers
  unsigned long long v_free[kNV];   // tcgen05.commit
  unsigned long long p_full[2];     // 8 softmax warps of CTA 0 (remote arrivals, each expecting its 4 KB bulk copy)
  unsigned long long corr_done[2];  // 4 correction warps
  unsigned long long pv_done[2];    // tcgen05.commit
  unsigned long long fin;           // 8 softmax warps of CTA 0: 1/l is in place
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int pad;
  float alpha[3][128];              // rescale factor of the tile (two buffers) and the final 1/l
};
static_assert(sizeof(Misc0) <= 4096 && sizeof(Misc1) <= 4096, "misc area");
static_assert(kOff1Misc + 4096 + 1024 <= kSmemBytes, "CTA 1 layout fits");

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Four rows (indices r0..r3) x 64 columns starting at column `col` -> 512 contiguous bytes of shared memory.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* tmap, uint32_t bar, int col, int r0, int r1, int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// remote arrival that also announces `bytes` of bulk-copy traffic to the barrier of another CTA of the cluster
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
// bulk copy local shared memory -> shared memory of another CTA; completes (byte count) on that CTA's barrier
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src_cta), "r"(bytes), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the bulk stores of this thread have read their shared-memory source (the global writes
// themselves complete before the grid does)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) sparse_mla_duo2_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                                                                       const __grid_constant__ CUtensorMap tm_o, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = static_cast<int>(cluster_ctarank());
  const int token = blockIdx.x >> 1;
  Misc0* m0 = reinterpret_cast<Misc0*>(sm + kOff0Misc);
  Misc1* m1 = reinterpret_cast<Misc1*>(sm + kOff1Misc);
  // abort_flag / n_scan / tmem_base sit at different offsets in the two layouts: pick this CTA's
  volatile int* abort_flag = cta == 0 ? &m0->abort_flag : &m1->abort_flag;
  int* n_scan_p = cta == 0 ? &m0->n_scan : &m1->n_scan;
  uint32_t* tmem_base_p = cta == 0 ? &m0->tmem_base : &m1->tmem_base;

  if (tid == 0) {
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    *n_scan_p = 0;
    if (cta == 0) {
      m0->bad_index = 0;
      for (int i = 0; i < kNK; ++i) { mbar_init(smem_u32(&m0->k_full[i]), 1); mbar_init(smem_u32(&m0->k_free[i]), 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&m0->s_full[i]), 1);
        mbar_init(smem_u32(&m0->s_free[i]), 8);
        mbar_init(smem_u32(&m0->p_free[i]), 1);
      }
      mbar_init(smem_u32(&m0->q_full), 1);
    } else {
      for (int i = 0; i < kNV; ++i) { mbar_init(smem_u32(&m1->v_full[i]), 1); mbar_init(smem_u32(&m1->v_free[i]), 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&m1->p_full[i]), 8);
        mbar_init(smem_u32(&m1->corr_done[i]), 4);
        mbar_init(smem_u32(&m1->pv_done[i]), 1);
      }
      mbar_init(smem_u32(&m1->fin), 8);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (*abort_flag) return;   // an earlier launch failed: both CTAs read the same status word

  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_base_p), 512u);
    tmem_relinquish();
    tc_fence_before();
  }
  if (cta == 0 && tid == 0) {
    // Q first, so that the loads run under the index scan below
    const uint32_t qf = smem_u32(&m0->q_full);
    mbar_arrive_expect_tx(qf, static_cast<uint32_t>(kNChunk * p.h * 128));
#pragma unroll 1
    for (int c = 0; c < kNChunk; ++c) tma_load_3d(base + c * kKSlot, &tm_q, qf, c * 64, 0, token);
  }
  const int32_t* idx_row = p.indices + static_cast<long long>(token) * p.idx_st;
  {
    int local = 0;
    for (int j = tid; j < p.topk; j += kThreads)
      if (idx_row[j] >= 0) local = j + 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = max(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0 && local > 0) atomicMax(n_scan_p, local);
  }
  if (cta == 0) {
    // Q goes to ring slots 0-8 (one 64-column block per slot, same 128B-swizzled layout as a K block) by
    // nine TMA tile loads of [h rows x 64 columns]; head rows h..127 of the slots are zeroed by hand.
    if (p.h < 128) {
      const int per_blk = (128 - p.h) * 8;
      for (int x = tid; x < kNChunk * per_blk; x += kThreads) {
        const int c = x / per_blk, y = x - c * per_blk;
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + c * kKSlot + p.h * 128 + y * 16), "r"(0) : "memory");
      }
    }
  }
  __syncthreads();
  tc_fence_after();
  if (cta == 0 && warp < 4) {
    // shared memory -> TMEM: thread = head row; a 32-bit TMEM column holds two consecutive bf16 of the row
    mbar_wait(smem_u32(&m0->q_full), 0u, abort_flag);
    const uint32_t tq = tmem_addr(*tmem_base_p, warp * 32, kColQ);
#pragma unroll 1
    for (int cc = 0; cc < kNChunk; ++cc) {
      uint32_t v[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t src = base + cc * kKSlot + tid * 128 + ((c ^ (tid & 7)) << 4);
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v[4 * c]), "=r"(v[4 * c + 1]), "=r"(v[4 * c + 2]), "=r"(v[4 * c + 3]) : "r"(src));
      }
      tmem_st32(tq + cc * 32, v);
    }
    tmem_wait_st();
    tc_fence_before();
    fence_proxy_async_smem();   // the ring slots read above are next written by TMA (async proxy)
  }
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_p;
  const int n_tiles = (*n_scan_p + kNT - 1) / kNT;

  if (cta == 0) {
    // ======================================================================= CTA 0: scores
    const uint32_t k_s = base + kOff0K;
    if (warp < 8) {
      // ---------------------------------------------------------------- softmax (two threads per head row)
      // thread tid: head row = tid % 128 (TMEM lane), columns 64*(tid/128) .. +63 of the tile.  Two passes
      // over TMEM (maximum, then exponentials) keep the register count low.
      const int rowi = tid & 127;
      const int ch = tid >> 7;
      const uint32_t p_remote = mapa_shared(base + kOff1P, 1);
      const uint32_t p_local = base + kOff0P;
      const uint32_t alpha_remote = mapa_shared(smem_u32(&m1->alpha[0][0]), 1);
      const uint32_t p_full_r[2] = {mapa_shared(smem_u32(&m1->p_full[0]), 1), mapa_shared(smem_u32(&m1->p_full[1]), 1)};
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
      float m_run = -INFINITY, l_run = 0.0f;
      for (int i = 0; i < n_tiles; ++i) {
        const int b = i & 1;
        mbar_wait(smem_u32(&m0->s_full[0]), i & 1u, abort_flag);
        tc_fence_after();
        const uint32_t vmA = m0->valid_mask[i & 3][2 * ch], vmB = m0->valid_mask[i & 3][2 * ch + 1];
        const bool all_valid = (m0->valid_mask[i & 3][0] & m0->valid_mask[i & 3][1] & m0->valid_mask[i & 3][2] &
                                m0->valid_mask[i & 3][3]) == 0xffffffffu;      // uniform over the CTA
        // copy this thread's 64 scores to registers and hand the single S buffer back at once
        uint32_t sr[2][32];
        const uint32_t t_s = tmem_addr(tmem, lane_base, kColS + ch * 64);
        tmem_ld32(t_s, sr[0]);
        tmem_ld32(t_s + 32, sr[1]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&m0->s_free[0]));
        float mx = -INFINITY;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (all_valid) {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(sr[q][j]));
          } else {
            const uint32_t vm = q == 0 ? vmA : vmB;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if ((vm >> j) & 1u) mx = fmaxf(mx, __uint_as_float(sr[q][j]));
          }
        }
        m0->xchg[b][tid] = mx;
        named_bar_sync(2, 256);
        mx = fmaxf(mx, m0->xchg[b][tid ^ 128]);
        // Lazy maximum: only move the reference when it grows by more than 2^8, so that the
        // accumulator in the other CTA is rarely rescaled (P stays below 256, exact enough in bf16/fp32).
        const float m_cand = fmaxf(m_run, mx * p.scale_log2);
        float alpha = 1.0f;
        if (m_cand > m_run + 8.0f || m_run == -INFINITY) {
          alpha = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_cand);
          m_run = m_cand;
        }
        const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
        // P buffer b of CTA 1 was last read by P.V of tile i-2
        if (i >= 2) mbar_wait(smem_u32(&m0->p_free[b]), ((i - 2) >> 1) & 1u, abort_flag);
        float psum = 0.0f;
        // this thread's 64 columns are block `ch` of the P buffer: row rowi, eight 16-byte chunks.  The
        // staging buffer b was last sent for tile i-2, whose P.V (awaited above) came after its arrival.
        const uint32_t p_row = p_local + b * kPBuf + ch * kQBlock + rowi * 128;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t vm = all_valid ? 0xffffffffu : (q == 0 ? vmA : vmB);
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float a0 = fast_exp2(fmaf(__uint_as_float(sr[q][j]), p.scale_log2, -m_use));
            float a1 = fast_exp2(fmaf(__uint_as_float(sr[q][j + 1]), p.scale_log2, -m_use));
            if (!all_valid) {
              a0 = ((vm >> j) & 1u) ? a0 : 0.0f;
              a1 = ((vm >> (j + 1)) & 1u) ? a1 : 0.0f;
            }
            psum += a0 + a1;
            pk[j >> 1] = pack_bf16x2(a0, a1);
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = q * 4 + c;
            st_shared_v4(p_row + ((chunk ^ (rowi & 7)) << 4), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          }
        }
        l_run = l_run * alpha + psum;
        if (ch == 0) st_cluster_f32(alpha_remote + (b * 128 + rowi) * 4, alpha);
        fence_proxy_async_smem();   // the bulk copy reads this warp's rows through the async proxy
        __syncwarp();
        if (lane == 0) {
          // this warp's 32 rows of block ch are 4 KB in a row, here and in CTA 1
          const uint32_t off = b * kPBuf + ch * kQBlock + lane_base * 128;
          mbar_arrive_expect_tx_cluster(p_full_r[b], 32 * 128);
          bulk_copy_to_cluster(p_remote + off, p_local + off, 32 * 128, p_full_r[b]);
        }
      }
      // final: combine the two halves of every row sum; 1/l goes to the other CTA, LSE is written here
      named_bar_sync(2, 256);
      m0->xchg[0][tid] = l_run;
      named_bar_sync(2, 256);
      const float l_tot = l_run + m0->xchg[0][tid ^ 128];
      if (ch == 0) {
        const float inv_l = (l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
        st_cluster_f32(alpha_remote + (2 * 128 + rowi) * 4, inv_l);
        if (rowi < p.h) {
          float v = -INFINITY;
          if (l_tot > 0.0f) {
            const float l2 = m_run + log2f(l_tot);
            v = p.lse_base2 ? l2 : l2 * 0.6931471805599453f;
          }
          p.lse[static_cast<long long>(token) * p.lse_st + rowi] = v;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&m1->fin), 1));
    } else if (warp == 8) {
      // ---------------------------------------------------------------- Q.K^T issuer
      // Straight-line code per tile (the ring holds exactly one tile, so block c always sits in slot c):
      // the descriptors differ in their low word only and every offset is a compile-time constant.
      static_assert(kNK == kNChunk, "slot index = column block index");
      if (lane == 0) {
        constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, kNT, 0, 0);
        const uint64_t bd0 = smem_desc_sw128(k_s, 16, 1024);
        const uint32_t bd_lo = static_cast<uint32_t>(bd0), bd_hi = static_cast<uint32_t>(bd0 >> 32);
        const uint32_t t_s = tmem + kColS, t_q = tmem + kColQ;
        const uint32_t k_full0 = smem_u32(&m0->k_full[0]), k_free0 = smem_u32(&m0->k_free[0]);
        const uint32_t s_full = smem_u32(&m0->s_full[0]), s_free = smem_u32(&m0->s_free[0]);
        for (int i = 0; i < n_tiles; ++i) {
          const uint32_t ph = i & 1u;
          // the single S buffer: the softmax of tile i-1 has copied it to registers
          if (i >= 1) mbar_wait(s_free, ph ^ 1u, abort_flag);
#pragma unroll
          for (int cc = 0; cc < kNChunk; ++cc) {
            mbar_wait(k_full0 + cc * 8, ph, abort_flag);
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t lo = bd_lo + ((cc * kKSlot + k * 32) >> 4);
              if (cc == 0 && k == 0) umma_f16_ts_lohi<false>(t_s, t_q + cc * 32 + k * 8, lo, bd_hi, kIdesc);
              else umma_f16_ts_lohi<true>(t_s, t_q + cc * 32 + k * 8, lo, bd_hi, kIdesc);
            }
            umma_commit(k_free0 + cc * 8);
          }
          umma_commit(s_full);
        }
      }
    } else {
      // ---------------------------------------------------------------- K producers (warps 9-17)
      // warp 9+c fetches 64-column block c of every tile; lane l owns tile rows 4l..4l+3 (one gather4).
      const int c = warp - 9;
      int nxt[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) nxt[j] = (4 * lane + j < p.topk) ? idx_row[4 * lane + j] : -1;
      for (int i = 0; i < n_tiles; ++i) {
        int row[4];
        uint32_t nib = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool ok = nxt[j] >= 0 && nxt[j] < p.s_kv;
          if (c == 0 && nxt[j] >= p.s_kv) m0->bad_index = 1;
          row[j] = ok ? nxt[j] : 0;
          nib |= ok ? (1u << j) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int jn = (i + 1) * kNT + 4 * lane + j;
          nxt[j] = (i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
        }
        if (c == 0) {
          // 128 validity bits of the tile: word w = rows 32w..32w+31 = lanes 8w..8w+7, four bits each
          uint32_t v = nib << ((lane & 7) * 4);
          v |= __shfl_xor_sync(0xffffffffu, v, 1);
          v |= __shfl_xor_sync(0xffffffffu, v, 2);
          v |= __shfl_xor_sync(0xffffffffu, v, 4);
          if ((lane & 7) == 0) m0->valid_mask[i & 3][lane >> 3] = v;
        }
        const int g = i * kNChunk + c;
        const int slot = g % kNK;
        if (g >= kNK) mbar_wait(smem_u32(&m0->k_free[slot]), ((g / kNK) - 1) & 1u, abort_flag);
        const uint32_t full = smem_u32(&m0->k_full[slot]);
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(full, kKSlot);
        __syncwarp();
        tma_gather4(k_s + slot * kKSlot + lane * 512, &tm_kv, full, c * 64, row[0], row[1], row[2], row[3]);
      }
    }
  } else {
    // ======================================================================= CTA 1: values
    const uint32_t v_s = base;
    const uint32_t p_s = base + kOff1P;
    if (warp < 8) {
      if (warp < 4) {
        // -------------------------------------------------------------- correction (thread = head)
        for (int i = 0; i < n_tiles; ++i) {
          const int b = i & 1;
          mbar_wait(smem_u32(&m1->p_full[b]), (i >> 1) & 1u, abort_flag);
          const float a = m1->alpha[b][tid];
          const bool need = (i > 0) && (a != 1.0f);
          if (__any_sync(0xffffffffu, need)) {
            mbar_wait(smem_u32(&m1->pv_done[(i - 1) & 1]), ((i - 1) >> 1) & 1u, abort_flag);
            tc_fence_after();
#pragma unroll 1
            for (int c0 = 0; c0 < 512; c0 += 32) {
              uint32_t o[32];
              tmem_ld32(tmem_addr(tmem, warp * 32, c0), o);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * a);
              tmem_st32(tmem_addr(tmem, warp * 32, c0), o);
            }
            tmem_wait_st();
            tc_fence_before();
          }
          // P arrived through the async proxy (bulk copy), which is also how the MMA reads it: no proxy fence
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&m1->corr_done[b]));
        }
      } else if (warp == 4 && lane == 0) {
        // -------------------------------------------------------------- relay: P buffer free -> CTA 0
        const uint32_t p_free_r[2] = {mapa_shared(smem_u32(&m0->p_free[0]), 0), mapa_shared(smem_u32(&m0->p_free[1]), 0)};
        for (int i = 0; i + 2 < n_tiles; ++i) {
          mbar_wait(smem_u32(&m1->pv_done[i & 1]), (i >> 1) & 1u, abort_flag);
          mbar_arrive_cluster(p_free_r[i & 1]);
        }
      }
      __syncwarp();
      // ---------------------------------------------------------------- epilogue (8 warps)
      // warp w: head rows 32*(w%4) .. +31 (its TMEM lanes), output columns 256*(w/4) .. +255.  The V ring
      // and the P buffers are idle once the last P.V has completed; O is staged there as bf16 rows of
      // 1024 + 16 bytes and each thread sends its 512-byte half row with one bulk store.
      // `fin` first: warps 4-7 arrive here before the first tile, and a parity wait is only exact once the
      // barrier is in, or past, the phase waited for (after `fin` the P.V of tile n-3 has completed)
      mbar_wait(smem_u32(&m1->fin), 0u, abort_flag);
      if (n_tiles > 0) {
        mbar_wait(smem_u32(&m1->pv_done[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1u, abort_flag);
        tc_fence_after();
      }
      const int row = (warp & 3) * 32 + lane;
      const int half = warp >> 2;
      const float inv_l = m1->alpha[2][row];
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        uint32_t acc[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem_addr(tmem, (warp & 3) * 32, half * 256 + c0), acc);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        // 64-column block cb of the staging area: [128 rows x 128 B], 16-byte chunks XOR-swizzled by row % 8
        const int cb = half * 4 + (c0 >> 6);
        const uint32_t o_blk = base + cb * kQBlock + row * 128;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          const int chunk = ((c0 & 63) + j) >> 3;
          st_shared_v4(o_blk + ((chunk ^ (row & 7)) << 4),
                       pack_bf16x2(__uint_as_float(acc[j]) * inv_l, __uint_as_float(acc[j + 1]) * inv_l),
                       pack_bf16x2(__uint_as_float(acc[j + 2]) * inv_l, __uint_as_float(acc[j + 3]) * inv_l),
                       pack_bf16x2(__uint_as_float(acc[j + 4]) * inv_l, __uint_as_float(acc[j + 5]) * inv_l),
                       pack_bf16x2(__uint_as_float(acc[j + 6]) * inv_l, __uint_as_float(acc[j + 7]) * inv_l));
        }
      }
      fence_proxy_async_smem();   // the tile stores read the staging area through the async proxy
      named_bar_sync(5, 256);
      if (lane == 0) {
        // warp w stores 64-column block w: one TMA tile store of [h rows x 64 columns]
        tma_store_3d(&tm_o, base + warp * kQBlock, warp * 64, 0, token);
        bulk_commit();
        bulk_wait_read_all();
      }
      tc_fence_before();
    } else if (warp == 8) {
      // ---------------------------------------------------------------- P.V issuer
      static_assert(kNV == kNT / kVSlabRows, "slab index = ring slot index");
      if (lane == 0) {
        constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, 256, 0, 1);
        const uint64_t ad0 = smem_desc_sw128(p_s, 16, 1024);
        const uint64_t bd0 = smem_desc_sw128(v_s, kVBlock, 1024);
        const uint32_t ad_lo = static_cast<uint32_t>(ad0), ad_hi = static_cast<uint32_t>(ad0 >> 32);
        const uint32_t bd_lo = static_cast<uint32_t>(bd0), bd_hi = static_cast<uint32_t>(bd0 >> 32);
        const uint32_t v_full0 = smem_u32(&m1->v_full[0]), v_free0 = smem_u32(&m1->v_free[0]);
        for (int i = 0; i < n_tiles; ++i) {
          const int b = i & 1;
          const uint32_t ph = i & 1u;
          mbar_wait(smem_u32(&m1->corr_done[b]), (i >> 1) & 1u, abort_flag);
          tc_fence_after();
          const uint32_t a_lo = ad_lo + ((b * kPBuf) >> 4);
#pragma unroll
          for (int sl = 0; sl < kNV; ++sl) {
            mbar_wait(v_full0 + sl * 8, ph, abort_flag);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int j = sl * 2 + kk;   // 16-row step inside the tile
              const uint32_t alo = a_lo + (((j >> 2) * kQBlock + (j & 3) * 32) >> 4);
#pragma unroll
              for (int hv = 0; hv < 2; ++hv) {
                const uint32_t blo = bd_lo + ((sl * kVSlab + hv * 4 * kVBlock + kk * 2048) >> 4);
                if (j == 0) {
                  if (i == 0) umma_f16_ss_lohi<false>(tmem + hv * 256, alo, ad_hi, blo, bd_hi, kIdesc);
                  else umma_f16_ss_lohi<true>(tmem + hv * 256, alo, ad_hi, blo, bd_hi, kIdesc);
                } else {
                  umma_f16_ss_lohi<true>(tmem + hv * 256, alo, ad_hi, blo, bd_hi, kIdesc);
                }
              }
            }
            umma_commit(v_free0 + sl * 8);
          }
          umma_commit(smem_u32(&m1->pv_done[b]));
        }
      }
    } else if (warp >= 9 && warp < 17) {
      // ---------------------------------------------------------------- V producers (warps 9-16)
      // warp 9+w fetches 64-column block w of the 512 value columns; lane l owns tile rows 4l..4l+3, which
      // are rows 4(l%8).. of slab l/8.
      const int w = warp - 9;
      const int sl = lane >> 3;
      int nxt[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) nxt[j] = (4 * lane + j < p.topk) ? idx_row[4 * lane + j] : -1;
      for (int i = 0; i < n_tiles; ++i) {
        int row[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) row[j] = (nxt[j] >= 0 && nxt[j] < p.s_kv) ? nxt[j] : 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int jn = (i + 1) * kNT + 4 * lane + j;
          nxt[j] = (i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
        }
        const int g = i * (kNT / kVSlabRows) + sl;
        const int slot = g % kNV;
        if (g >= kNV) mbar_wait(smem_u32(&m1->v_free[slot]), ((g / kNV) - 1) & 1u, abort_flag);
        const uint32_t full = smem_u32(&m1->v_full[slot]);
        // one arrival per slab announces all 64 gathers of the eight warps (the byte count may run
        // ahead of the announcement: the phase cannot complete before this arrival)
        if (w == 0 && (lane & 7) == 0) mbar_arrive_expect_tx(full, kVSlab);
        tma_gather4(v_s + slot * kVSlab + w * kVBlock + (lane & 7) * 512, &tm_kv, full, w * 64, row[0], row[1], row[2], row[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // nobody leaves while the peer may still write or signal this CTA
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512u);
  }
  if (tid == 0 && p.status != nullptr) {
    if (*abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
    else if (cta == 0 && m0->bad_index) atomicCAS(p.status, 0, FTB_ERR_BAD_INDEX);
  }
}

}  // namespace mla4

int launch_sparse_mla_duo2(const ftb_sparse_mla_args* a, cudaStream_t st) {
  mla4::Params p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.kv = reinterpret_cast<const __nv_bfloat16*>(a->kv);
  p.indices = a->indices;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.s_q = a->s_q; p.h = a->h; p.s_kv = a->s_kv; p.topk = a->topk;
  p.q_st = a->q_stride_token; p.q_sh = a->q_stride_head; p.kv_sr = a->kv_stride_row;
  p.idx_st = a->idx_stride_token; p.out_st = a->out_stride_token; p.out_sh = a->out_stride_head;
  p.lse_st = a->lse_stride_token;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f;
  p.lse_base2 = a->lse_base2;
  p.status = a->status;
  // box = 64 columns x 1 row: tile::gather4 fetches four such rows per instruction
  CUtensorMap tm_kv;
  if (!make_tmap_2d(&tm_kv, a->kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(a->s_kv), mla4::kDqk,
                    static_cast<uint64_t>(a->kv_stride_row), 1, 64)) {
    set_last_error("sparse_mla_duo2: cuTensorMapEncodeTiled failed");
    return FTB_ERR_CUDA;
  }
  const uint32_t box_h = static_cast<uint32_t>(a->h < 128 ? a->h : 128);
  CUtensorMap tm_q, tm_o;
  if (!make_tmap_3d(&tm_q, a->q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, mla4::kDqk, static_cast<uint64_t>(a->h),
                    static_cast<uint64_t>(a->s_q), static_cast<uint64_t>(a->q_stride_head),
                    static_cast<uint64_t>(a->q_stride_token), 64, box_h) ||
      !make_tmap_3d(&tm_o, a->out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 512, static_cast<uint64_t>(a->h),
                    static_cast<uint64_t>(a->s_q), static_cast<uint64_t>(a->out_stride_head),
                    static_cast<uint64_t>(a->out_stride_token), 64, box_h)) {
    set_last_error("sparse_mla_duo2: cuTensorMapEncodeTiled failed for q or out");
    return FTB_ERR_CUDA;
  }
  cudaError_t e = cudaFuncSetAttribute(mla4::sparse_mla_duo2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla4::kSmemBytes);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla_duo)");
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(a->s_q) * 2u);
  cfg.blockDim = dim3(mla4::kThreads);
  cfg.dynamicSmemBytes = mla4::kSmemBytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, mla4::sparse_mla_duo2_kernel, tm_kv, tm_q, tm_o, p);
  return check_cuda(e, "sparse_mla_duo launch");
}

}  // namespace ftb
