// Top-k sparse MLA forward, persistent role-split CTA pairs (bf16 KV), one ring for K and Q.
//
// One pair of CTAs (a cluster of 2) walks through query tokens pair, pair + pairs, ...  CTA 0 computes
// S = Q.K^T (Q in tensor memory, K column blocks from a ring in shared memory filled by TMA gather4) and the
// softmax; P travels to CTA 1 by bulk copies over distributed shared memory; CTA 1 accumulates O += P.V in
// tensor memory and writes the output.  Every barrier keeps counting across tokens.
//
// The ring of CTA 0.  Eleven slots of [128 rows x 128 B] hold a stream of entries that the MMA issuer
// consumes strictly in order: per token nine Q entries (the 64-column blocks of the token's query rows,
// fetched by a TMA tile load and moved on to tensor memory by the issuer itself with tcgen05.cp, which runs
// in order with its MMAs) and then nine K entries per tile of 128 selected rows (one 64-column block
// each, fetched by one warp with a 32-lane gather4, multiplied by four MMAs).  Entry n lives in slot n % 11.
// A tile needs nine slots, so two entries of look-ahead remain: a slot is refilled from the moment its
// MMAs (or its copy to tensor memory) have completed, and the time that takes, about 5000 cycles in the kernel
// with a nine-slot ring against 2300 cycles of MMAs per tile, is what bounds the tile period; each further slot
// takes 256 cycles off it.  The room for the two slots comes from a single staging buffer for P.  The next
// token's Q needs no special case: its entries follow the last tile's in the ring, its loads go out while
// the last tile is still being multiplied (and the token after it is asked into L2), and no warp has to
// carry Q from shared to tensor memory.
//
// Gather warps.  A warp hands the TMA unit one gather4 every 65 to 70 cycles, lane after lane (a 32-lane
// instruction keeps it busy for 2240 cycles, 16 lanes for 1260), and warps that share a scheduler share its
// dispatch of such operations (about one per 20 cycles per scheduler).  So every K entry belongs to two warps, 16
// lanes and 64 rows each, eighteen gather warps in all, and they sit on the three schedulers that the MMA
// issuer is not on (warp ids 9-31 except those that are 0 modulo 4): with four gather warps beside it the
// issuer needed 420 instead of 265 cycles per block.
// The kernel runs 32 warps per CTA; registers move from the gather warps to the softmax / correction warps
// (setmaxnreg), and every group of warps runs its own copy of the batch loop so that its budget applies to its
// own code only.
//
// Softmax: two threads per head row; the running maximum moves only when it grows by more than 2^8, so that
// the accumulator in CTA 1 is rarely rescaled.  P (bf16) and the rescale factors go to a staging area and
// from there to CTA 1 with bulk copies that complete on CTA 1's barrier; the arrival that announces them
// carries no release (the data travels with the copies), which keeps the softmax warps from stalling.
//
// The number of tiles of a token (last non-negative index, rounded up to 128 rows, at least one) is
// found for 64 tokens at a time by all warps of a CTA, with a CTA barrier on either side.
//
// Warps (1024 threads per CTA): CTA 0: 0-7 softmax, 8 MMA issuer, eighteen ring producers (producer 2c + hf: rows
// 64 hf .. 64 hf + 63 of block c of every tile; hf = 0 also loads block c of Q).  CTA 1: 0-3 correction, 4 relay,
// 8 MMA issuer, 9-16 V producers, 0-7 and 9-16 epilogue.
// Every wait is bounded; a wait that runs out sets the abort flag, after which every later wait returns at
// once and the status word reports a timeout.
#include <type_traits>

#include "sm100.cuh"
#include "tmap.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace mla_ring {

constexpr int kDqk = 576;
constexpr int kNChunk = 9;
constexpr int kNT = 128;                       // gathered rows per tile
constexpr int kQBlock = 128 * 128;             // 16384: [128 heads x 128 B]
constexpr int kNK = 11;                        // ring slots of CTA 0: entry n (a Q block or a K block of a tile) lives in slot n % 11
constexpr int kKSlot = kNT * 128;              // 16384: [128 rows x 128 B]
constexpr int kNV = 4;                         // V ring slots: one whole tile, slab s in slot s
constexpr int kVSlabRows = 32;
constexpr int kVBlock = kVSlabRows * 128;      // 4096: one 64-column block of a slab
constexpr int kVSlab = 8 * kVBlock;            // 32768
constexpr int kPBuf = 2 * kQBlock;             // 32768: P [128 heads x 128 rows] bf16 as two 64-row blocks
constexpr int kBatch = 64;                     // tokens whose tile counts are found in one go
// CTA 0 layout: ring of 11 slots | P staging | misc.
// CTA 1 layout: V ring | P x 2 | misc; between tokens the P buffer of the last tile stages O.
constexpr int kOff0K = 0;
constexpr int kOff0P = kOff0K + kNK * kKSlot;              // 180224
constexpr int kOff0Misc = kOff0P + kPBuf;                  // 212992
constexpr int kOff1P = kNV * kVSlab;                       // 131072
constexpr int kOff1Misc = kOff1P + 2 * kPBuf;              // 196608
constexpr int kSmemBytes = kOff0Misc + 4096 + 1024;        // the larger of the two + misc + alignment slack
constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr uint32_t kColQ = 0;                  // TMEM columns of CTA 0: Q (288), then S
constexpr uint32_t kColS = 320;

struct Params {
  const int32_t* indices;
  float* lse;
  int s_q, h, s_kv, topk;
  long long idx_st, lse_st;
  float scale_log2;
  int lse_base2;
  int* status;
};

struct Misc0 {   // CTA 0
  unsigned long long k_full[kNK];   // two arrivals, one per gather warp of the entry, each announcing its bytes (8 KB of gathers; the tile load of a Q entry counts on the first)
  unsigned long long k_free[kNK];   // tcgen05.commit behind the entry's MMAs or its copy to tensor memory
  unsigned long long s_full;        // tcgen05.commit
  unsigned long long s_free;        // 8 softmax warps
  unsigned long long p_free[2];     // relay warp of CTA 1 (remote arrival)
  unsigned long long stage_free;    // correction warp 0 of CTA 1 (remote arrival): P and the factors of the tile have landed there
  unsigned long long epi_done[2];   // CTA 1 (remote arrival): the epilogue of token t (t % 2) is over
  uint32_t tmem_base;
  int abort_flag;
  int bad_index;
  int pad;
  uint32_t valid_mask[4][4];        // per tile (mod 4): 128 validity bits
  unsigned short nt[kBatch];        // tiles per token of the current batch
  float xchg[2][256];               // row maximum / row sum exchange between the two threads of a head row
  alignas(16) float alpha_stage[128]; // rescale factors of a tile on their way to CTA 1 (sent with P)
};
struct Misc1 {   // CTA 1
  unsigned long long v_full[kNV];   // one arrival announcing 32 KB of gathers
  unsigned long long v_free[kNV];   // tcgen05.commit
  unsigned long long p_full[2];     // 8 softmax warps of CTA 0 (remote arrivals, each announcing its bulk copies: 4 KB of P, 128 B of factors)
  unsigned long long corr_done[2];  // 4 correction warps
  unsigned long long pv_done[2];    // tcgen05.commit
  unsigned long long fin[2];        // 8 softmax warps of CTA 0: 1/l of token t (t % 2) is in place
  unsigned long long o_free;        // 16 epilogue warps: the accumulator has been read
  unsigned long long stg_free[8];   // epilogue warp w < 8: its staging piece is free for warp 9 + w
  unsigned long long epi_cnt;       // 16 epilogue warps: the output of the token has left the staging area
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
  unsigned short nt[kBatch];
  alignas(16) float alpha[2][128];  // rescale factor of the tile (two buffers), written by bulk copies from CTA 0
  float inv_l[2][128];              // final 1/l of token t (t % 2)
};
static_assert(sizeof(Misc0) <= 4096 && sizeof(Misc1) <= 4096, "misc area");
static_assert(kOff1Misc + 4096 + 1024 <= kSmemBytes, "CTA 1 layout fits");
static_assert(kNV == kNT / kVSlabRows, "V ring slot index = slab index");
static_assert(kNK > kNChunk && kNK < 2 * kNChunk, "a ring position advances by one tile with a single wrap test");

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
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// remote arrival that also announces `bytes` of bulk-copy traffic to the barrier of another CTA of the cluster.
// No release: what the waiter reads arrives with the announced copies themselves.  (With release semantics at
// cluster scope this arrival stalled the softmax warps for about 2000 cycles per tile.)
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
// remote arrival that only hands a buffer back (nothing the waiter reads depends on it)
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// shared memory -> tensor memory, 128 rows x 32 bytes (one K = 16 step of an A operand), asynchronous and in order
// with the MMAs of the issuing thread; the source is described like an MMA operand
__device__ __forceinline__ void tmem_cp_128x256b(uint32_t taddr, uint32_t desc_lo, uint32_t desc_hi) {
  asm volatile(
      "{\n\t.reg .b64 sd;\n\t"
      "mov.b64 sd, {%1, %2};\n\t"
      "tcgen05.cp.cta_group::1.128x256b [%0], sd;\n\t}"
      ::"r"(taddr), "r"(desc_lo), "r"(desc_hi)
      : "memory");
}
// position of a role in the stream of ring entries: slot = n % kNK, use = n / kNK
struct RingPos {
  uint32_t slot, use;
  __device__ __forceinline__ void advance(uint32_t by) {   // by < kNK
    slot += by;
    if (slot >= static_cast<uint32_t>(kNK)) { slot -= kNK; ++use; }
  }
};
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

__global__ void __launch_bounds__(kThreads, 1)
sparse_mla_ring_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                         const __grid_constant__ CUtensorMap tm_o, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = static_cast<int>(cluster_ctarank());
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  Misc0* m0 = reinterpret_cast<Misc0*>(sm + kOff0Misc);
  Misc1* m1 = reinterpret_cast<Misc1*>(sm + kOff1Misc);
  // abort_flag / tmem_base / nt sit at different offsets in the two layouts: pick this CTA's
  volatile int* abort_flag = cta == 0 ? &m0->abort_flag : &m1->abort_flag;
  uint32_t* tmem_base_p = cta == 0 ? &m0->tmem_base : &m1->tmem_base;
  unsigned short* nt = cta == 0 ? m0->nt : m1->nt;

  if (tid == 0) {
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    if (cta == 0) {
      m0->bad_index = 0;
      for (int i = 0; i < kNK; ++i) { mbar_init(smem_u32(&m0->k_full[i]), 2); mbar_init(smem_u32(&m0->k_free[i]), 1); }
      mbar_init(smem_u32(&m0->s_full), 1);
      mbar_init(smem_u32(&m0->s_free), 8);
      for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&m0->p_free[i]), 1); mbar_init(smem_u32(&m0->epi_done[i]), 1); }
      mbar_init(smem_u32(&m0->stage_free), 1);
    } else {
      for (int i = 0; i < kNV; ++i) { mbar_init(smem_u32(&m1->v_full[i]), 1); mbar_init(smem_u32(&m1->v_free[i]), 1); }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&m1->p_full[i]), 8);
        mbar_init(smem_u32(&m1->corr_done[i]), 4);
        mbar_init(smem_u32(&m1->pv_done[i]), 1);
        mbar_init(smem_u32(&m1->fin[i]), 8);
      }
      mbar_init(smem_u32(&m1->o_free), 16);
      for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&m1->stg_free[i]), 1);
      mbar_init(smem_u32(&m1->epi_cnt), 16);
    }
    fence_mbar_init();
  }
  __syncthreads();
  cluster_sync_all();
  // An earlier launch on this status word failed: leave at once.  The two CTAs of a pair read the word at
  // different moments (another pair of this launch may report in between), so CTA 1 takes CTA 0's reading:
  // a CTA that went on alone would signal barriers in the shared memory of a partner that has left.
  {
    uint32_t leave;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(leave) : "r"(mapa_shared(smem_u32(&m0->abort_flag), 0)) : "memory");
    if (leave != 0u) {
      cluster_sync_all();      // CTA 0 stays until its partner has read the flag
      return;
    }
    __syncthreads();
    if (tid == 0) *abort_flag = 0;
  }
  if (cta == 0 && p.h < 128) {
    // a Q entry only writes h rows of its slot; the rows below feed head rows that are never stored, but they
    // should hold numbers
    for (int x = tid; x < kNK * kKSlot / 16; x += kThreads)
      asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + x * 16), "r"(0) : "memory");
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_base_p), 512u);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_p;
  // tokens of this pair: pair, pair + n_pairs, ...  (the host launches no more pairs than tokens)
  const int my_tokens = (p.s_q - pair + n_pairs - 1) / n_pairs;
  uint32_t gt = 0;   // tiles processed before the current token: every role counts the same way
  // CTA 0: index of this warp among the eighteen ring producers (-1 = not one): the warps 9-31 whose id is not 0
  // modulo 4, in order (they share no scheduler with the MMA issuer, warp 8).
  const int prod = (warp >= 9 && (warp & 3) != 0) ? (warp - 9) - ((warp - 8) >> 2) : -1;
  RingPos pos;       // CTA 0, issuer and producers: position in the stream of ring entries
  pos.slot = (cta == 0 && prod >= 0) ? static_cast<uint32_t>(prod >> 1) : 0u;
  pos.use = 0;

  // The body of the kernel as a function of the warp group it is compiled for (0: warps 0-7, 1: warps 8-19,
  // 2: warps 20-31): every group runs the same batch loop, but each copy only holds its own roles, so that the
  // register budget set for the group applies to exactly the code that the group executes.
  auto run = [&](auto group_tag) {
  constexpr int GRP = decltype(group_tag)::value;
  for (int batch0 = 0; batch0 < my_tokens; batch0 += kBatch) {
    const int nb = min(kBatch, my_tokens - batch0);
    // ------------------------------------------------------------------ tiles per token of this batch
    for (int t = warp; t < nb; t += kWarps) {
      const int tok = pair + (batch0 + t) * n_pairs;
      const int32_t* idx_row = p.indices + static_cast<long long>(tok) * p.idx_st;
      int local = 0;
      for (int j = lane; j < p.topk; j += 32)
        if (idx_row[j] >= 0) local = j + 1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) local = max(local, __shfl_xor_sync(0xffffffffu, local, o));
      // at least one tile (entirely masked if the token selects nothing): every stage of the pipeline
      // then runs once per token and the hand-overs between tokens need no special case
      if (lane == 0) nt[t] = static_cast<unsigned short>(min(65535, max(1, (local + kNT - 1) / kNT)));
    }
    __syncthreads();

    if (cta == 0) {
      // ===================================================================== CTA 0: scores
      const uint32_t k_s = base + kOff0K;
      if constexpr (GRP == 0) {
        // -------------------------------------------------------------- softmax (two threads per head row)
        // thread tid: head row = tid % 128 (TMEM lane), columns 64*(tid/128) .. +63 of the tile
        const int rowi = tid & 127;
        const int ch = tid >> 7;
        const uint32_t p_remote = mapa_shared(base + kOff1P, 1);
        const uint32_t p_local = base + kOff0P;
        const uint32_t alpha_remote = mapa_shared(smem_u32(&m1->alpha[0][0]), 1);
        const uint32_t invl_remote = mapa_shared(smem_u32(&m1->inv_l[0][0]), 1);
        const uint32_t p_full_r[2] = {mapa_shared(smem_u32(&m1->p_full[0]), 1), mapa_shared(smem_u32(&m1->p_full[1]), 1)};
        const uint32_t fin_r[2] = {mapa_shared(smem_u32(&m1->fin[0]), 1), mapa_shared(smem_u32(&m1->fin[1]), 1)};
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
        for (int t = 0; t < nb; ++t) {
          const int ti = batch0 + t;
          const int tok = pair + ti * n_pairs;
          const int n_tiles = nt[t];
          // 1/l and the `fin` barrier of parity ti % 2 were last used by token ti - 2: its epilogue is over
          if (ti >= 2) mbar_wait(smem_u32(&m0->epi_done[ti & 1]), ((ti >> 1) - 1) & 1u, abort_flag);
          float m_run = -INFINITY, l_run = 0.0f;
          for (int i = 0; i < n_tiles; ++i) {
            const uint32_t G = gt + i;
            const int b = G & 1;
            mbar_wait(smem_u32(&m0->s_full), G & 1u, abort_flag);
            tc_fence_after();
            const uint32_t vmA = m0->valid_mask[G & 3][2 * ch], vmB = m0->valid_mask[G & 3][2 * ch + 1];
            const bool all_valid = (m0->valid_mask[G & 3][0] & m0->valid_mask[G & 3][1] & m0->valid_mask[G & 3][2] &
                                    m0->valid_mask[G & 3][3]) == 0xffffffffu;      // uniform over the CTA
            // copy this thread's 64 scores to registers and hand the single S buffer back at once
            uint32_t sr[2][32];
            const uint32_t t_s = tmem_addr(tmem, lane_base, kColS + ch * 64);
            tmem_ld32(t_s, sr[0]);
            tmem_ld32(t_s + 32, sr[1]);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&m0->s_free));
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
            // P buffer b of CTA 1 was last read by P.V of tile G-2
            if (G >= 2) mbar_wait(smem_u32(&m0->p_free[b]), ((G - 2) >> 1) & 1u, abort_flag);
            // the staging area is single: CTA 1 reports as soon as the copies of the tile before have landed
            if (G >= 1) mbar_wait(smem_u32(&m0->stage_free), (G - 1) & 1u, abort_flag);
            float psum = 0.0f;
            // this thread's 64 columns are block `ch` of the P buffer: row rowi, eight 16-byte chunks
            const uint32_t p_row = p_local + ch * kQBlock + rowi * 128;
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
            if (ch == 0) m0->alpha_stage[rowi] = alpha;
            fence_proxy_async_smem();   // the bulk copies read this warp's rows through the async proxy
            __syncwarp();
            if (lane == 0) {
              // this warp's 32 rows of block ch are 4 KB in a row, here and in CTA 1; the warps of block 0 also
              // send the rescale factors of their 32 rows
              const uint32_t off = ch * kQBlock + lane_base * 128;
              mbar_arrive_expect_tx_cluster(p_full_r[b], 32 * 128 + (ch == 0 ? 128 : 0));
              bulk_copy_to_cluster(p_remote + b * kPBuf + off, p_local + off, 32 * 128, p_full_r[b]);
              if (ch == 0)
                bulk_copy_to_cluster(alpha_remote + (b * 128 + lane_base) * 4, smem_u32(&m0->alpha_stage[lane_base]), 128, p_full_r[b]);
            }
          }
          gt += n_tiles;
          // end of the token: combine the two halves of every row sum; 1/l goes to CTA 1, LSE is written here
          named_bar_sync(2, 256);
          m0->xchg[0][tid] = l_run;
          named_bar_sync(2, 256);
          const float l_tot = l_run + m0->xchg[0][tid ^ 128];
          named_bar_sync(2, 256);   // xchg[0] may be written again by the first tile of the next token
          if (ch == 0) {
            const float inv_l = (l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
            st_cluster_f32(invl_remote + ((ti & 1) * 128 + rowi) * 4, inv_l);
            if (rowi < p.h) {
              float v = -INFINITY;
              if (l_tot > 0.0f) {
                const float l2 = m_run + log2f(l_tot);
                v = p.lse_base2 ? l2 : l2 * 0.6931471805599453f;
              }
              p.lse[static_cast<long long>(tok) * p.lse_st + rowi] = v;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(fin_r[ti & 1]);
        }
      } else if (GRP == 1 && warp == 8) {
        // -------------------------------------------------------------- ring consumer: Q copies and Q.K^T
        // The whole warp runs the loop and waits; an elected lane (always the same one, so that its commits
        // cover its MMAs and copies) issues.  The descriptors differ in their low word only.  Per token: nine Q
        // entries, each moved to its 32 columns of tensor memory by four tcgen05.cp (they run in order behind
        // the MMAs issued before them, so the previous token's last tile has read the block by then), then nine K
        // entries per tile with four MMAs each.  The commit behind an entry frees its slot.
        {
          constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, kNT, 0, 0);
          const uint64_t bd0 = smem_desc_sw128(k_s, 16, 1024);
          const uint32_t bd_lo = static_cast<uint32_t>(bd0), bd_hi = static_cast<uint32_t>(bd0 >> 32);
          const uint32_t t_s = tmem + kColS, t_q = tmem + kColQ;
          const uint32_t k_full0 = smem_u32(&m0->k_full[0]), k_free0 = smem_u32(&m0->k_free[0]);
          const uint32_t s_full = smem_u32(&m0->s_full), s_free = smem_u32(&m0->s_free);
          for (int t = 0; t < nb; ++t) {
            const int n_tiles = nt[t];
#pragma unroll 1
            for (int cc = 0; cc < kNChunk; ++cc) {
              mbar_wait(k_full0 + pos.slot * 8, pos.use & 1u, abort_flag);
              tc_fence_after();
              if (elect_one()) {
                const uint32_t lo = bd_lo + ((pos.slot * kKSlot) >> 4);
#pragma unroll
                for (int k = 0; k < 4; ++k) tmem_cp_128x256b(t_q + cc * 32 + k * 8, lo + ((k * 32) >> 4), bd_hi);
                umma_commit(k_free0 + pos.slot * 8);
              }
              __syncwarp();
              pos.advance(1);
            }
            for (int i = 0; i < n_tiles; ++i) {
              const uint32_t G = gt + i;
              // the single S buffer: the softmax of tile G-1 has copied it to registers
              if (G >= 1) mbar_wait(s_free, (G & 1u) ^ 1u, abort_flag);
#pragma unroll
              for (int cc = 0; cc < kNChunk; ++cc) {
                mbar_wait(k_full0 + pos.slot * 8, pos.use & 1u, abort_flag);
                tc_fence_after();
                if (elect_one()) {
                  const uint32_t lo = bd_lo + ((pos.slot * kKSlot) >> 4);
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    if (cc == 0 && k == 0) umma_f16_ts_lohi<false>(t_s, t_q + cc * 32 + k * 8, lo + ((k * 32) >> 4), bd_hi, kIdesc);
                    else umma_f16_ts_lohi<true>(t_s, t_q + cc * 32 + k * 8, lo + ((k * 32) >> 4), bd_hi, kIdesc);
                  }
                  umma_commit(k_free0 + pos.slot * 8);
                }
                __syncwarp();
                pos.advance(1);
              }
              if (elect_one()) umma_commit(s_full);
              __syncwarp();
            }
            gt += n_tiles;
          }
        }
      } else if (prod >= 0) {
        // -------------------------------------------------------------- ring producers
        // producer 2c + hf supplies rows 64 hf .. 64 hf + 63 of block c of every tile (lane l < 16 owns tile rows
        // 64 hf + 4l .. + 3: one gather4) and, if hf = 0, block c of every token's Q (one TMA tile load), in the
        // order of the ring: its entries are c, c + 9, c + 18, ...  A slot is free once the commit behind the
        // entry that used it last has arrived (k_free); the parity wait is exact because the entry eleven places
        // back is at most one phase away.  Each of the two warps of an entry arrives on its barrier with its own
        // byte count.  Block c of the token after this one is asked into L2 when this token's is loaded.
        const int c = prod >> 1, hf = prod & 1;
        const bool glane = lane < 16;
        const int r0 = 64 * hf + 4 * (lane & 15);
        for (int t = 0; t < nb; ++t) {
          const int ti = batch0 + t;
          const int tok = pair + ti * n_pairs;
          const int n_tiles = nt[t];
          const int32_t* idx_row = p.indices + static_cast<long long>(tok) * p.idx_st;
          int nxt[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) nxt[j] = (glane && r0 + j < p.topk) ? idx_row[r0 + j] : -1;
          // ---- the Q entry
          if (pos.use >= 1) mbar_wait(smem_u32(&m0->k_free[pos.slot]), (pos.use - 1) & 1u, abort_flag);
          if (lane == 0) {
            const uint32_t full = smem_u32(&m0->k_full[pos.slot]);
            if (hf == 0) {
              mbar_arrive_expect_tx(full, static_cast<uint32_t>(p.h * 128));
              tma_load_3d(k_s + pos.slot * kKSlot, &tm_q, full, c * 64, 0, tok);
              if (tok + n_pairs < p.s_q)
                asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                             ::"l"(&tm_q), "r"(c * 64), "r"(0), "r"(tok + n_pairs) : "memory");
            } else {
              mbar_arrive(full);
            }
          }
          __syncwarp();
          pos.advance(kNChunk);
          // ---- the K entries
          for (int i = 0; i < n_tiles; ++i) {
            const uint32_t G = gt + i;
            int row[4];
            uint32_t nib = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const bool ok = nxt[j] >= 0 && nxt[j] < p.s_kv;
              if (c == 0 && (nxt[j] >= p.s_kv || nxt[j] < -1)) m0->bad_index = 1;
              row[j] = ok ? nxt[j] : 0;
              nib |= ok ? (1u << j) : 0u;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int jn = (i + 1) * kNT + r0 + j;
              nxt[j] = (glane && i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
            }
            if (c == 0) {
              // 64 validity bits of this half of the tile: word 2 hf + w = rows 64 hf + 32w .. + 31 = lanes 8w .. 8w + 7
              uint32_t v = glane ? (nib << ((lane & 7) * 4)) : 0u;
              v |= __shfl_xor_sync(0xffffffffu, v, 1);
              v |= __shfl_xor_sync(0xffffffffu, v, 2);
              v |= __shfl_xor_sync(0xffffffffu, v, 4);
              if (glane && (lane & 7) == 0) m0->valid_mask[G & 3][2 * hf + (lane >> 3)] = v;
            }
            if (pos.use >= 1) mbar_wait(smem_u32(&m0->k_free[pos.slot]), (pos.use - 1) & 1u, abort_flag);
            const uint32_t full = smem_u32(&m0->k_full[pos.slot]);
            __syncwarp();
            if (lane == 0) mbar_arrive_expect_tx(full, kKSlot / 2);
            __syncwarp();
            if (glane) tma_gather4(k_s + pos.slot * kKSlot + r0 * 128, &tm_kv, full, c * 64, row[0], row[1], row[2], row[3]);
            pos.advance(kNChunk);
          }
          gt += n_tiles;
        }
      }
    } else {
      // ===================================================================== CTA 1: values
      const uint32_t v_s = base;
      const uint32_t p_s = base + kOff1P;
      const uint32_t epi_done_r[2] = {mapa_shared(smem_u32(&m0->epi_done[0]), 0), mapa_shared(smem_u32(&m0->epi_done[1]), 0)};
      // ---------------------------------------------------------------- epilogue duty (16 warps: 0-7 and 9-16)
      // warp -> TMEM lane quarter warp % 4 (head rows 32q .. 32q+31) and column group g (output columns
      // 128g .. 128g+127): warps 0-3 g = 0, 4-7 g = 1, 9-12 g = 2, 13-16 g = 3.  A warp works alone: it
      // converts 64 columns of its rows to bf16 into a private 4 KB piece of the P buffer of the token's
      // last tile ([32 rows x 128 B], the swizzled tile layout) and sends it with one TMA tile store, twice.
      // That P buffer is idle until the softmax two tiles later asks for it, and the relay holds its
      // p_free back until the last store has read it; the V ring is not touched, so the gathers of the
      // next token run underneath.  Warp w < 8 and warp 9 + w share piece w: the V producers come later
      // (they first send out the next token's first gathers) and wait for their partner (stg_free).
      auto epilogue_duty = [&](int ti, uint32_t Gl, int tok) {
        const int q4 = warp & 3;
        const int grp = warp < 8 ? (warp >> 2) : 2 + ((warp - 9) >> 2);
        const int piece = warp < 8 ? warp : warp - 9;
        // `fin` first: a parity wait is only exact once the barrier is in, or past, the phase waited for
        // (after `fin` the P.V two tiles before the last one has completed)
        mbar_wait(smem_u32(&m1->fin[ti & 1]), (ti >> 1) & 1u, abort_flag);
        mbar_wait(smem_u32(&m1->pv_done[Gl & 1]), (Gl >> 1) & 1u, abort_flag);
        if (warp >= 9) mbar_wait(smem_u32(&m1->stg_free[piece]), ti & 1u, abort_flag);
        tc_fence_after();
        const int row = q4 * 32 + lane;
        const float inv_l = m1->inv_l[ti & 1][row];
        const uint32_t stg = p_s + (Gl & 1u) * kPBuf + piece * 4096 + lane * 128;
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t acc[32];
            tmem_ld32(tmem_addr(tmem, q4 * 32, grp * 128 + cb * 64 + c2 * 32), acc);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int chunk = c2 * 4 + (j >> 3);
              st_shared_v4(stg + ((chunk ^ (lane & 7)) << 4),
                           pack_bf16x2(__uint_as_float(acc[j]) * inv_l, __uint_as_float(acc[j + 1]) * inv_l),
                           pack_bf16x2(__uint_as_float(acc[j + 2]) * inv_l, __uint_as_float(acc[j + 3]) * inv_l),
                           pack_bf16x2(__uint_as_float(acc[j + 4]) * inv_l, __uint_as_float(acc[j + 5]) * inv_l),
                           pack_bf16x2(__uint_as_float(acc[j + 6]) * inv_l, __uint_as_float(acc[j + 7]) * inv_l));
            }
          }
          if (cb == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&m1->o_free));   // the next token's P.V may overwrite the accumulator
          }
          fence_proxy_async_smem();   // the tile store reads the piece through the async proxy
          __syncwarp();
          if (lane == 0) {
            if (q4 * 32 < p.h) tma_store_3d(&tm_o, stg - lane * 128, (grp * 2 + cb) * 64, q4 * 32, tok);
            bulk_commit();
            bulk_wait_read_all();
          }
          __syncwarp();
        }
        if (lane == 0) {
          if (warp < 8) mbar_arrive(smem_u32(&m1->stg_free[piece]));
          mbar_arrive(smem_u32(&m1->epi_cnt));
        }
      };
      if constexpr (GRP == 0) {
        const uint32_t p_free_r[2] = {mapa_shared(smem_u32(&m0->p_free[0]), 0), mapa_shared(smem_u32(&m0->p_free[1]), 0)};
        const uint32_t stage_free_r = mapa_shared(smem_u32(&m0->stage_free), 0);
        for (int t = 0; t < nb; ++t) {
          const int ti = batch0 + t;
          const int tok = pair + ti * n_pairs;
          const int n_tiles = nt[t];
          if (warp < 4) {
            // ------------------------------------------------------------ correction (thread = head)
            for (int i = 0; i < n_tiles; ++i) {
              const uint32_t G = gt + i;
              const int b = G & 1;
              mbar_wait(smem_u32(&m1->p_full[b]), (G >> 1) & 1u, abort_flag);
              if (tid == 0) mbar_arrive_cluster_relaxed(stage_free_r);   // the copies have read CTA 0's staging area
              const float a = m1->alpha[b][tid];
              const bool need = (i > 0) && (a != 1.0f);
              if (__any_sync(0xffffffffu, need)) {
                mbar_wait(smem_u32(&m1->pv_done[(G - 1) & 1]), ((G - 1) >> 1) & 1u, abort_flag);
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
            // ------------------------------------------------------------ relay: P buffer free -> CTA 0
            for (int i = 0; i + 1 < n_tiles; ++i) {
              const uint32_t G = gt + i;
              mbar_wait(smem_u32(&m1->pv_done[G & 1]), (G >> 1) & 1u, abort_flag);
              mbar_arrive_cluster_relaxed(p_free_r[G & 1]);
            }
          }
          __syncwarp();
          gt += n_tiles;
          epilogue_duty(ti, gt - 1, tok);
          // the P buffer of the last tile staged the output: it is free for the softmax, and 1/l of this
          // token may be replaced, once all 16 warps are through
          if (warp == 4 && lane == 0) {
            mbar_wait(smem_u32(&m1->epi_cnt), ti & 1u, abort_flag);
            mbar_arrive_cluster_relaxed(p_free_r[(gt - 1) & 1]);
            mbar_arrive_cluster_relaxed(epi_done_r[ti & 1]);
          }
        }
      } else if (GRP == 1 && warp == 8) {
        // -------------------------------------------------------------- P.V issuer (whole warp, an elected lane issues)
        {
          constexpr uint32_t kIdesc = umma_idesc(kFmtBF16, 128, 256, 0, 1);
          const uint64_t ad0 = smem_desc_sw128(p_s, 16, 1024);
          const uint64_t bd0 = smem_desc_sw128(v_s, kVBlock, 1024);
          const uint32_t ad_lo = static_cast<uint32_t>(ad0), ad_hi = static_cast<uint32_t>(ad0 >> 32);
          const uint32_t bd_lo = static_cast<uint32_t>(bd0), bd_hi = static_cast<uint32_t>(bd0 >> 32);
          const uint32_t v_full0 = smem_u32(&m1->v_full[0]), v_free0 = smem_u32(&m1->v_free[0]);
          for (int t = 0; t < nb; ++t) {
            const int ti = batch0 + t;
            const int n_tiles = nt[t];
            // the epilogue of the previous token has read the accumulator
            if (ti >= 1) mbar_wait(smem_u32(&m1->o_free), (ti - 1) & 1u, abort_flag);
            for (int i = 0; i < n_tiles; ++i) {
              const uint32_t G = gt + i;
              const int b = G & 1;
              const uint32_t ph = G & 1u;
              mbar_wait(smem_u32(&m1->corr_done[b]), (G >> 1) & 1u, abort_flag);
              tc_fence_after();
              const uint32_t a_lo = ad_lo + ((b * kPBuf) >> 4);
#pragma unroll
              for (int sl = 0; sl < kNV; ++sl) {
                mbar_wait(v_full0 + sl * 8, ph, abort_flag);
                tc_fence_after();
                if (elect_one()) {
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
                __syncwarp();
              }
              if (elect_one()) umma_commit(smem_u32(&m1->pv_done[b]));
              __syncwarp();
            }
            gt += n_tiles;
          }
        }
      } else if (warp >= 9 && warp < 17) {
        // -------------------------------------------------------------- V producers (warps 9-16)
        // warp 9+w fetches 64-column block w of the 512 value columns; lane l owns tile rows 4l..4l+3, which
        // are rows 4(l%8).. of slab l/8.
        const int w = warp - 9;
        const int sl = lane >> 3;
        for (int t = 0; t < nb; ++t) {
          const int ti = batch0 + t;
          const int tok = pair + ti * n_pairs;
          const int n_tiles = nt[t];
          const int32_t* idx_row = p.indices + static_cast<long long>(tok) * p.idx_st;
          int nxt[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) nxt[j] = (4 * lane + j < p.topk) ? idx_row[4 * lane + j] : -1;
          auto issue_tile = [&](int i) {
            const uint32_t G = gt + i;
            int row[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) row[j] = (nxt[j] >= 0 && nxt[j] < p.s_kv) ? nxt[j] : 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int jn = (i + 1) * kNT + 4 * lane + j;
              nxt[j] = (i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
            }
            if (G >= 1) mbar_wait(smem_u32(&m1->v_free[sl]), (G - 1) & 1u, abort_flag);
            const uint32_t full = smem_u32(&m1->v_full[sl]);
            // one arrival per slab announces all 64 gathers of the eight warps (the byte count may run
            // ahead of the announcement: the phase cannot complete before this arrival)
            if (w == 0 && (lane & 7) == 0) mbar_arrive_expect_tx(full, kVSlab);
            tma_gather4(v_s + sl * kVSlab + w * kVBlock + (lane & 7) * 512, &tm_kv, full, w * 64, row[0], row[1], row[2], row[3]);
          };
          // the first tile goes out before this warp helps with the previous token's epilogue, so that the
          // gathers run underneath it
          issue_tile(0);
          __syncwarp();
          if (t > 0) epilogue_duty(ti - 1, gt - 1, tok - n_pairs);
          for (int i = 1; i < n_tiles; ++i) issue_tile(i);
          gt += n_tiles;
        }
        // the last token of the batch: nothing of the next batch is known yet
        __syncwarp();
        epilogue_duty(batch0 + nb - 1, gt - 1, pair + (batch0 + nb - 1) * n_pairs);
      }
    }
    __syncthreads();   // nt[] is rewritten by the next batch
  }
  };
  // Registers follow the work: the gather warps need few, the softmax and correction / epilogue warps many
  // (64 scores per thread live at once).
  if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
    run(std::integral_constant<int, 0>{});
  } else if (warp < 20) {
    run(std::integral_constant<int, 1>{});
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    run(std::integral_constant<int, 2>{});
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

}  // namespace mla_ring

int launch_sparse_mla_ring(const ftb_sparse_mla_args* a, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(mla_ring::sparse_mla_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla_ring::kSmemBytes);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla_ring)");
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(mla_ring::kThreads);
  cfg.dynamicSmemBytes = mla_ring::kSmemBytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // as many pairs as the device holds at once (one per pair of SMs that can host a cluster), cached per device
  static int pairs_of_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int pairs_dev = (dev >= 0 && dev < 64) ? pairs_of_device[dev] : 0;
  if (pairs_dev == 0) {
    cfg.gridDim = dim3(2);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, mla_ring::sparse_mla_ring_kernel, &cfg);
    if (e != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      int sms = 0;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      n = sms / 2 > 0 ? sms / 2 : 1;
    }
    pairs_dev = n;
    if (dev >= 0 && dev < 64) pairs_of_device[dev] = pairs_dev;
  }
  // One launch takes at most kBatch tokens per pair, so that every pair finds its tile counts once and runs
  // through its tokens without a stop; a longer batch of query tokens is a sequence of such launches on the
  // stream (a launch boundary every pairs x kBatch tokens costs next to nothing).
  const long long cap = static_cast<long long>(pairs_dev) * mla_ring::kBatch;
  // KV: box = 64 columns x 1 row (tile::gather4 fetches four such rows per instruction);
  // Q: boxes of [h rows x 64 columns] of one token; O: boxes of [32 rows x 64 columns] (a store that
  // reaches past row h is clipped)
  const uint32_t box_h = static_cast<uint32_t>(a->h < 128 ? a->h : 128);
  CUtensorMap tm_kv;
  if (!make_tmap_2d(&tm_kv, a->kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(a->s_kv), mla_ring::kDqk,
                    static_cast<uint64_t>(a->kv_stride_row), 1, 64)) {
    set_last_error("sparse_mla_ring: cuTensorMapEncodeTiled failed");
    return FTB_ERR_CUDA;
  }
  for (long long t0 = 0; t0 < a->s_q; t0 += cap) {
    const int n_tok = static_cast<int>(a->s_q - t0 < cap ? a->s_q - t0 : cap);
    mla_ring::Params p;
    p.indices = a->indices + t0 * a->idx_stride_token;
    p.lse = a->lse + t0 * a->lse_stride_token;
    p.s_q = n_tok; p.h = a->h; p.s_kv = a->s_kv; p.topk = a->topk;
    p.idx_st = a->idx_stride_token;
    p.lse_st = a->lse_stride_token;
    p.scale_log2 = a->sm_scale * 1.4426950408889634f;
    p.lse_base2 = a->lse_base2;
    p.status = a->status;
    const void* q0 = static_cast<const __nv_bfloat16*>(a->q) + t0 * a->q_stride_token;
    void* o0 = static_cast<__nv_bfloat16*>(a->out) + t0 * a->out_stride_token;
    CUtensorMap tm_q, tm_o;
    if (!make_tmap_3d(&tm_q, q0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, mla_ring::kDqk, static_cast<uint64_t>(a->h),
                      static_cast<uint64_t>(n_tok), static_cast<uint64_t>(a->q_stride_head),
                      static_cast<uint64_t>(a->q_stride_token), 64, box_h) ||
        !make_tmap_3d(&tm_o, o0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 512, static_cast<uint64_t>(a->h),
                      static_cast<uint64_t>(n_tok), static_cast<uint64_t>(a->out_stride_head),
                      static_cast<uint64_t>(a->out_stride_token), 64, box_h < 32 ? box_h : 32)) {
      set_last_error("sparse_mla_ring: cuTensorMapEncodeTiled failed");
      return FTB_ERR_CUDA;
    }
    const int pairs = pairs_dev < n_tok ? pairs_dev : n_tok;
    cfg.gridDim = dim3(static_cast<unsigned>(pairs) * 2u);
    e = cudaLaunchKernelEx(&cfg, mla_ring::sparse_mla_ring_kernel, tm_kv, tm_q, tm_o, p);
    if (e != cudaSuccess) return check_cuda(e, "sparse_mla_ring launch");
  }
  return FTB_OK;
}

}  // namespace ftb
