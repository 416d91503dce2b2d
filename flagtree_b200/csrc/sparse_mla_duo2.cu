// Top-k sparse MLA forward, role-split CTA pair with Q held in tensor memory (bf16 KV).
//
// Same division of labour as sparse_mla_duo.cu (CTA 0: S = Q.K^T + softmax, CTA 1: O += P.V, P sent over
// distributed shared memory) with one change that matters for the K ring: Q [128 heads x 576] is not kept
// in shared memory (147 KB) but in CTA 0's tensor memory (288 of 512 columns, two bf16 per 32-bit column)
// and enters the MMA as the TMEM A operand.  That frees the shared memory for a 13-slot ring of K column
// blocks (208 KB) instead of 4 slots, so the gather runs far ahead of the MMAs.  TMEM of CTA 0: Q in
// columns 0-287, one S buffer [128 x 128] in columns 320-447 (the softmax copies S to registers at once,
// so one buffer is enough).
//
// Warps (544 threads per CTA): CTA 0: 0-7 softmax (two threads per head row), 8 MMA issuer, 9-16 K producers.
// CTA 1: 0-3 correction + epilogue, 4 relay, 8 MMA issuer, 9-16 V producers.  Every wait is bounded.
#include "sm100.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace mla4 {

constexpr int kDqk = 576;
constexpr int kNChunk = 9;
constexpr int kNT = 128;                       // gathered rows per tile
constexpr int kQBlock = 128 * 128;             // 16384: [128 heads x 128 B]
constexpr int kQBytes = kNChunk * kQBlock;     // 147456
constexpr int kNK = 13;                        // K ring slots (Q lives in TMEM)
constexpr int kKSlot = kNT * 128;              // 16384: [128 rows x 128 B]
constexpr int kNV = 4;                         // V ring slots
constexpr int kVSlabRows = 32;
constexpr int kVBlock = kVSlabRows * 128;      // 4096: one 64-column block of a slab
constexpr int kVSlab = 8 * kVBlock;            // 32768
constexpr int kPBuf = 2 * kQBlock;             // 32768: P [128 heads x 128 rows] bf16 as two 64-row blocks
// CTA 0 layout: K ring | misc (Q is staged in ring slots 0-8 once, then moved to TMEM).
// CTA 1 layout: V ring | P x 2 | misc.
constexpr int kOff0K = 0;
constexpr int kOff0Misc = kOff0K + kNK * kKSlot;           // 212992
constexpr int kOff1P = kNV * kVSlab;                       // 131072
constexpr int kOff1Misc = kOff1P + 2 * kPBuf;              // 196608
constexpr int kSmemBytes = kOff0Misc + 4096 + 1024;        // the larger of the two + misc + alignment slack
constexpr int kThreads = 544;
constexpr uint32_t kColQ = 0;                  // TMEM columns of CTA 0: Q (288), then S
constexpr uint32_t kColS = 320;
constexpr int kProducers = 256;                // producer threads per CTA (warps 9-16)

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
  unsigned long long k_full[kNK];   // every producer thread, when its own copies have landed
  unsigned long long k_free[kNK];   // tcgen05.commit
  unsigned long long s_full[2];     // tcgen05.commit (index 0 used: one S buffer)
  unsigned long long s_free[2];     // 8 softmax warps (index 0 used)
  unsigned long long p_free[2];     // relay warp of CTA 1 (remote arrival)
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int bad_index;
  uint32_t valid_mask[4][4];        // per tile (mod 4): 128 validity bits
  int rows[2][kNT];
  float xchg[2][256];               // row maximum / row sum exchange between the two threads of a head row
};
struct Misc1 {   // CTA 1
  unsigned long long v_full[kNV];   // every producer thread, when its own copies have landed
  unsigned long long v_free[kNV];   // tcgen05.commit
  unsigned long long p_full[2];     // 8 softmax warps of CTA 0 (remote arrivals)
  unsigned long long corr_done[2];  // 4 correction warps
  unsigned long long pv_done[2];    // tcgen05.commit
  unsigned long long fin;           // 8 softmax warps of CTA 0: 1/l is in place
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int pad;
  float alpha[3][128];              // rescale factor of the tile (two buffers) and the final 1/l
  int rows[2][kNT];
};
static_assert(sizeof(Misc0) <= 4096 && sizeof(Misc1) <= 4096, "misc area");
static_assert(kOff1Misc + 4096 + 1024 <= kSmemBytes, "CTA 1 layout fits");

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void cp_async_wait2() { asm volatile("cp.async.wait_group 2;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1) sparse_mla_duo2_kernel(const Params p) {
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
      for (int i = 0; i < kNK; ++i) { mbar_init(smem_u32(&m0->k_full[i]), kProducers); mbar_init(smem_u32(&m0->k_free[i]), 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&m0->s_full[i]), 1);
        mbar_init(smem_u32(&m0->s_free[i]), 8);
        mbar_init(smem_u32(&m0->p_free[i]), 1);
      }
    } else {
      for (int i = 0; i < kNV; ++i) { mbar_init(smem_u32(&m1->v_full[i]), kProducers); mbar_init(smem_u32(&m1->v_free[i]), 1); }
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
    // Q -> ring slots 0-8 (one 64-column block per slot, same 128B-swizzled layout as a K block)
    const __nv_bfloat16* q_tok = p.q + static_cast<long long>(token) * p.q_st;
    for (int c = tid; c < 128 * (kDqk / 8); c += kThreads) {
      const int r = c / (kDqk / 8);
      const int ch = c - r * (kDqk / 8);
      const uint32_t dst = base + (ch >> 3) * kKSlot + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
      if (r < p.h) cp_async16(dst, q_tok + static_cast<long long>(r) * p.q_sh + ch * 8);
      else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
    }
    cp_async_commit();
    cp_async_wait_all();
  }
  __syncthreads();
  tc_fence_after();
  if (cta == 0 && warp < 4) {
    // shared memory -> TMEM: thread = head row; a 32-bit TMEM column holds two consecutive bf16 of the row
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
        // this thread's 64 columns are block `ch` of the P buffer: row rowi, eight 16-byte chunks
        const uint32_t p_row = p_remote + b * kPBuf + ch * kQBlock + rowi * 128;
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
            st_cluster_v4(p_row + ((chunk ^ (rowi & 7)) << 4), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          }
        }
        tc_fence_before();
        l_run = l_run * alpha + psum;
        if (ch == 0) st_cluster_f32(alpha_remote + (b * 128 + rowi) * 4, alpha);
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(p_full_r[b]);
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
      if (lane == 0) {
        constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, kNT, 0, 0);
        for (int i = 0; i < n_tiles; ++i) {
          const int b = i & 1;
          // the single S buffer: the softmax of tile i-1 has copied it to registers
          if (i >= 1) mbar_wait(smem_u32(&m0->s_free[0]), (i - 1) & 1u, abort_flag);
          tc_fence_after();
          // Two column blocks per synchronisation: the per-block barrier wait, proxy fence and commit cost
          // more issue time than the four 64-cycle MMAs of one block.
#pragma unroll 1
          for (int cc = 0; cc < kNChunk; cc += 2) {
            const int nb = (cc + 1 < kNChunk) ? 2 : 1;
            const int g0 = i * kNChunk + cc;
            for (int u = 0; u < nb; ++u) mbar_wait(smem_u32(&m0->k_full[(g0 + u) % kNK]), ((g0 + u) / kNK) & 1u, abort_flag);
            fence_proxy_async_smem();   // the copies were written through the generic proxy
            tc_fence_after();
            for (int u = 0; u < nb; ++u) {
              const int slot = (g0 + u) % kNK;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint64_t bd = smem_desc_sw128(k_s + slot * kKSlot + k * 32, 16, 1024);
                umma_f16_ts(tmem + kColS, tmem + kColQ + (cc + u) * 32 + k * 8, bd, kIdesc, ((cc + u) | k) != 0 ? 1u : 0u);
              }
              umma_commit(smem_u32(&m0->k_free[slot]));
            }
          }
          umma_commit(smem_u32(&m0->s_full[0]));
        }
      }
    } else {
      // ---------------------------------------------------------------- K producers (warps 9-16)
      const int pt = tid - 288;   // 0..255; the first 128 also resolve one tile slot each
      const int pw = warp - 9;    // rows pw*16 .. pw*16+15 of every block
      int idx_next = (pt < kNT && pt < p.topk) ? idx_row[pt] : -1;
      int g = 0;
      for (int i = 0; i < n_tiles; ++i) {
        if (pt < kNT) {
          const int logical = idx_next;
          const int jn = (i + 1) * kNT + pt;
          idx_next = (i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
          const bool ok = logical >= 0 && logical < p.s_kv;
          if (logical >= p.s_kv) m0->bad_index = 1;
          const uint32_t m = __ballot_sync(0xffffffffu, ok);
          if (lane == 0) m0->valid_mask[i & 3][pt >> 5] = m;
          m0->rows[i & 1][pt] = ok ? logical : 0;
        }
        named_bar_sync(3, kProducers);
        // this lane's 4 rows of every block: row = pw*16 + it*4 + lane/8, 16-byte chunk lane%8
        const __nv_bfloat16* src[4];
#pragma unroll
        for (int it = 0; it < 4; ++it)
          src[it] = p.kv + static_cast<long long>(m0->rows[i & 1][pw * 16 + it * 4 + (lane >> 3)]) * p.kv_sr + (lane & 7) * 8;
#pragma unroll 1
        for (int cc = 0; cc < kNChunk; ++cc, ++g) {
          const int slot = g % kNK;
          if (g >= kNK) mbar_wait(smem_u32(&m0->k_free[slot]), ((g / kNK) - 1) & 1u, abort_flag);
          const uint32_t dslot = k_s + slot * kKSlot;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int r = pw * 16 + it * 4 + (lane >> 3);
            cp_async16(dslot + r * 128 + (((lane & 7) ^ (r & 7)) << 4), src[it] + cc * 64);
          }
          // the barrier hears from this thread when the copies above have landed; the thread itself
          // does not wait and goes on to the next ring slot
          cp_async_mbar_arrive_noinc(smem_u32(&m0->k_full[slot]));
        }
      }
      cp_async_wait_all();
    }
  } else {
    // ======================================================================= CTA 1: values
    const uint32_t v_s = base;
    const uint32_t p_s = base + kOff1P;
    if (warp < 4) {
      // ---------------------------------------------------------------- correction + epilogue (thread = head)
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
        fence_proxy_async_all();     // P arrived through the generic proxy; the MMA reads it through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&m1->corr_done[b]));
      }
      if (n_tiles > 0) {
        mbar_wait(smem_u32(&m1->pv_done[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1u, abort_flag);
        tc_fence_after();
      }
      mbar_wait(smem_u32(&m1->fin), 0u, abort_flag);
      const float inv_l = m1->alpha[2][tid];
      __nv_bfloat16* orow = p.out + static_cast<long long>(token) * p.out_st + static_cast<long long>(tid) * p.out_sh;
#pragma unroll 1
      for (int c0 = 0; c0 < 512; c0 += 32) {
        uint32_t acc[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem_addr(tmem, warp * 32, c0), acc);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        if (tid < p.h) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(acc[j]) * inv_l, __uint_as_float(acc[j + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(acc[j + 2]) * inv_l, __uint_as_float(acc[j + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(acc[j + 4]) * inv_l, __uint_as_float(acc[j + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(acc[j + 6]) * inv_l, __uint_as_float(acc[j + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c0 + j) = v;
          }
        }
      }
      tc_fence_before();
    } else if (warp == 8) {
      // ---------------------------------------------------------------- P.V issuer
      if (lane == 0) {
        constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, 256, 0, 1);
        for (int i = 0; i < n_tiles; ++i) {
          const int b = i & 1;
          mbar_wait(smem_u32(&m1->corr_done[b]), (i >> 1) & 1u, abort_flag);
          tc_fence_after();
#pragma unroll 1
          for (int sl = 0; sl < kNT / kVSlabRows; ++sl) {
            const int g = i * (kNT / kVSlabRows) + sl;
            const int slot = g % kNV;
            mbar_wait(smem_u32(&m1->v_full[slot]), (g / kNV) & 1u, abort_flag);
            fence_proxy_async_smem();
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int j = sl * 2 + kk;   // 16-row step inside the tile
              const uint64_t ad = smem_desc_sw128(p_s + b * kPBuf + (j >> 2) * kQBlock + (j & 3) * 32, 16, 1024);
#pragma unroll
              for (int hv = 0; hv < 2; ++hv) {
                const uint64_t bd = smem_desc_sw128(v_s + slot * kVSlab + hv * 4 * kVBlock + kk * 2048, kVBlock, 1024);
                umma_f16_ss(tmem + hv * 256, ad, bd, kIdesc, (i | j) != 0 ? 1u : 0u);
              }
            }
            umma_commit(smem_u32(&m1->v_free[slot]));
          }
          umma_commit(smem_u32(&m1->pv_done[b]));
        }
      }
    } else if (warp == 4) {
      // ---------------------------------------------------------------- relay: P buffer free -> CTA 0
      if (lane == 0) {
        const uint32_t p_free_r[2] = {mapa_shared(smem_u32(&m0->p_free[0]), 0), mapa_shared(smem_u32(&m0->p_free[1]), 0)};
        for (int i = 0; i + 2 < n_tiles; ++i) {
          mbar_wait(smem_u32(&m1->pv_done[i & 1]), (i >> 1) & 1u, abort_flag);
          mbar_arrive_cluster(p_free_r[i & 1]);
        }
      }
    } else if (warp >= 9) {
      // ---------------------------------------------------------------- V producers (warps 9-16)
      const int pt = tid - 288;   // 0..255
      const int pw = warp - 9;    // rows pw*4 .. pw*4+3 of every slab
      int idx_next = (pt < kNT && pt < p.topk) ? idx_row[pt] : -1;
      int g = 0;
      for (int i = 0; i < n_tiles; ++i) {
        if (pt < kNT) {
          const int logical = idx_next;
          const int jn = (i + 1) * kNT + pt;
          idx_next = (i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
          m1->rows[i & 1][pt] = (logical >= 0 && logical < p.s_kv) ? logical : 0;
        }
        named_bar_sync(4, kProducers);
#pragma unroll 1
        for (int sl = 0; sl < kNT / kVSlabRows; ++sl, ++g) {
          const int slot = g % kNV;
          if (g >= kNV) mbar_wait(smem_u32(&m1->v_free[slot]), ((g / kNV) - 1) & 1u, abort_flag);
          const uint32_t dslab = v_s + slot * kVSlab;
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r = pw * 4 + rr;           // row inside the slab
            const __nv_bfloat16* src = p.kv + static_cast<long long>(m1->rows[i & 1][sl * kVSlabRows + r]) * p.kv_sr;
#pragma unroll
            for (int part = 0; part < 2; ++part) {
              const int q = part * 32 + lane;     // 16-byte chunk of the 1024-byte V row
              cp_async16(dslab + (q >> 3) * kVBlock + r * 128 + (((q & 7) ^ (r & 7)) << 4), src + q * 8);
            }
          }
          cp_async_mbar_arrive_noinc(smem_u32(&m1->v_full[slot]));
        }
      }
      cp_async_wait_all();
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
  e = cudaLaunchKernelEx(&cfg, mla4::sparse_mla_duo2_kernel, p);
  return check_cuda(e, "sparse_mla_duo launch");
}

}  // namespace ftb
