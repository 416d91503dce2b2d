// Top-k sparse MLA forward, CTA-pair version (cluster of 2, tcgen05 cta_group::2), bf16 KV.
//
// One CTA pair per query token.  CTA c holds 64 of the 128 heads of Q (73.7 KB instead of 147 KB), so
// there is room for double-buffered KV tiles and nothing is computed twice:
//   S = Q.K^T : M = 128 (64 heads per CTA), N = 64 gathered rows (32 gathered by each CTA), K = 576.
//   O += P.V  : M = 128, N = 256 per instruction (2 instructions), K = 64 rows.  The B operand of a
//               pair MMA is split along N: CTA c supplies 128 of every 256 output columns for ALL 64
//               rows of the tile, so each CTA also gathers its output columns of the peer's rows.
// TMEM per CTA ("2x2" layout of a pair MMA with 64 rows per CTA: row r, column j of an N-wide result
// sits in lane r + 64*(j >= N/2), column j mod N/2): S double-buffered 2 x 32 columns, O 256 columns.
//
// Warp roles per CTA (416 threads): warps 0-3 softmax / rescale / epilogue (thread = TMEM lane),
// warp 4 MMA issuer (even CTA only) and TMEM owner, warps 5-8 gather K tiles, warps 9-12 gather V tiles.
// K and V tiles live in separate 2-deep rings: a K stage is free as soon as Q.K^T of its tile has
// finished, a V stage when P.V has.  All waits are bounded.
#include "sm100.cuh"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace mla2 {

constexpr int kDqk = 576;
constexpr int kNChunk = 9;                  // 64-column blocks of a latent row
constexpr int kHeadsCta = 64;
constexpr int kNT = 64;                     // gathered rows per pair tile
constexpr int kRowsOwn = kNT / 2;           // rows whose K part this CTA gathers
constexpr int kQBlock = kHeadsCta * 128;    // 8192
constexpr int kQBytes = kNChunk * kQBlock;  // 73728
constexpr int kKBlock = kRowsOwn * 128;     // 4096
constexpr int kKStage = kNChunk * kKBlock;  // 36864
constexpr int kVBlock = kNT * 128;          // 8192
constexpr int kVStage = 4 * kVBlock;        // 32768: this CTA's 256 output columns of all 64 rows
constexpr int kPBytes = kHeadsCta * 128;    // 8192: P [64 heads x 64 rows] bf16
constexpr int kOffK = kQBytes;
constexpr int kOffV = kOffK + 2 * kKStage;
constexpr int kOffP = kOffV + 2 * kVStage;
constexpr int kOffMisc = kOffP + 2 * kPBytes;        // 229376
constexpr int kSmemBytes = 232448;                   // everything a CTA may have: 3072 B for Misc + alignment
constexpr int kThreads = 416;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256;

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

struct Misc {
  unsigned long long k_full[2];    // even CTA: both CTAs' K rows of the stage have landed (8 warp arrivals)
  unsigned long long v_full[2];    // even CTA: both CTAs' V columns of the stage have landed (8 warp arrivals)
  unsigned long long p_full[2];    // even CTA: P written and O rescaled by all 8 softmax warps
  unsigned long long s_full[2];    // every CTA: Q.K^T of the tile finished (S readable, K stage free)
  unsigned long long pv_done[2];   // every CTA: P.V of the tile finished (V stage, P buffer free, O updated)
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int bad_index;
  uint32_t valid_mask[4][2];       // per tile (mod 4): validity of rows 0-31 / 32-63
  int k_rows[2][kRowsOwn];         // physical rows of this CTA's K rows, per K stage
  int v_rows[2][kNT];              // physical rows of all 64 rows, per V stage
  float xchg[128];                 // exchange between the two threads that share a head row
};
static_assert(sizeof(Misc) <= 2048, "Misc must fit behind the tiles even with 1023 bytes of alignment padding");

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void cp_async_wait_group1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_group0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1) sparse_mla_pair_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  Misc* misc = reinterpret_cast<Misc*>(sm + kOffMisc);
  volatile int* abort_flag = &misc->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int cta = static_cast<int>(cluster_ctarank());
  const int token = blockIdx.x >> 1;
  const uint32_t q_s = base;
  const uint32_t k_s = base + kOffK;
  const uint32_t v_s = base + kOffV;
  const uint32_t p_s = base + kOffP;

  if (tid == 0) {
    misc->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    misc->n_scan = 0;
    misc->bad_index = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&misc->k_full[i]), 8);
      mbar_init(smem_u32(&misc->v_full[i]), 8);
      mbar_init(smem_u32(&misc->p_full[i]), 8);
      mbar_init(smem_u32(&misc->s_full[i]), 1);
      mbar_init(smem_u32(&misc->pv_done[i]), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (misc->abort_flag) return;   // an earlier launch failed: both CTAs of the pair see the same word

  if (warp == 4) {
    tmem_alloc_pair(smem_u32(&misc->tmem_base), kTmemCols);
    tmem_relinquish_pair();
    tc_fence_before();
  }
  // last valid slot + 1 (both CTAs compute the same number)
  {
    int local = 0;
    const int32_t* idx_row = p.indices + static_cast<long long>(token) * p.idx_st;
    for (int j = tid; j < p.topk; j += kThreads)
      if (idx_row[j] >= 0) local = j + 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = max(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0 && local > 0) atomicMax(&misc->n_scan, local);
  }
  // Q rows of this CTA's 64 heads (rows beyond h are zero)
  {
    const __nv_bfloat16* q_tok = p.q + static_cast<long long>(token) * p.q_st;
    for (int c = tid; c < kHeadsCta * (kDqk / 8); c += kThreads) {
      const int r = c / (kDqk / 8);
      const int ch = c - r * (kDqk / 8);
      const uint32_t dst = q_s + (ch >> 3) * kQBlock + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
      const int head = cta * kHeadsCta + r;
      if (head < p.h) cp_async16(dst, q_tok + static_cast<long long>(head) * p.q_sh + ch * 8);
      else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
    }
    cp_async_commit();
    cp_async_wait_all();
    fence_proxy_async_smem();
  }
  __syncthreads();
  cluster_sync_all();            // barriers initialised, Q of both CTAs in place, TMEM allocated
  tc_fence_after();
  const uint32_t tmem = misc->tmem_base;
  const int n_tiles = (misc->n_scan + kNT - 1) / kNT;
  const int32_t* idx_row = p.indices + static_cast<long long>(token) * p.idx_st;

  if (warp < 4) {
    // ---------------------------------------------------------------- softmax / rescale / epilogue
    const int head_l = tid & 63;             // head within this CTA
    const int hh = tid >> 6;                 // which half of the tile's rows / of the output columns
    const uint32_t p_full0 = mapa_shared(smem_u32(&misc->p_full[0]), 0);
    const uint32_t p_full1 = mapa_shared(smem_u32(&misc->p_full[1]), 0);
    float m_run = -INFINITY, l_run = 0.0f;
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      mbar_wait(smem_u32(&misc->s_full[b]), (i >> 1) & 1u, abort_flag);
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, kColS + b * 32), sr);
      tmem_wait_ld();
      const uint32_t vm = misc->valid_mask[i & 3][hh];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if ((vm >> j) & 1u) mx = fmaxf(mx, __uint_as_float(sr[j]));
      misc->xchg[tid] = mx;
      named_bar_sync(2, 128);
      mx = fmaxf(mx, misc->xchg[tid ^ 64]);
      named_bar_sync(2, 128);               // everyone has read before the next write
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_use);
      float psum = 0.0f;
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float a0 = ((vm >> j) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[j]), p.scale_log2, -m_use)) : 0.0f;
        const float a1 = ((vm >> (j + 1)) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[j + 1]), p.scale_log2, -m_use)) : 0.0f;
        psum += a0 + a1;
        pk[j >> 1] = pack_bf16x2(a0, a1);
      }
      l_run = l_run * alpha + psum;
      m_run = m_new;
      // P buffer b was last read by P.V of tile i-2
      if (i >= 2) mbar_wait(smem_u32(&misc->pv_done[b]), ((i - 2) >> 1) & 1u, abort_flag);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t dst = p_s + b * kPBytes + head_l * 128 + (((hh * 4 + c) ^ (head_l & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                     "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                     : "memory");
      }
      // rescale O when a row maximum moved; P.V of tile i-1 must have finished first
      const bool need = (i > 0) && (alpha != 1.0f);
      if (__any_sync(0xffffffffu, need)) {
        mbar_wait(smem_u32(&misc->pv_done[(i - 1) & 1]), ((i - 1) >> 1) & 1u, abort_flag);
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_addr(tmem, warp * 32, kColO + c0), o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st32(tmem_addr(tmem, warp * 32, kColO + c0), o);
        }
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(b ? p_full1 : p_full0);
    }
    // ---- epilogue
    if (n_tiles > 0) {
      mbar_wait(smem_u32(&misc->pv_done[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1u, abort_flag);
      tc_fence_after();
    }
    misc->xchg[tid] = l_run;
    named_bar_sync(2, 128);
    const float l_tot = l_run + misc->xchg[tid ^ 64];
    const float inv_l = (l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
    const int head = cta * kHeadsCta + head_l;
    __nv_bfloat16* orow = p.out + static_cast<long long>(token) * p.out_st + static_cast<long long>(head) * p.out_sh;
#pragma unroll 1
    for (int c0 = 0; c0 < 256; c0 += 32) {
      uint32_t acc[32];
      if (n_tiles > 0) {
        tmem_ld32(tmem_addr(tmem, warp * 32, kColO + c0), acc);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
      }
      if (head < p.h) {
        // TMEM column x of this lane half -> output column 256*(x/128) + 128*hh + x%128
        const int dv0 = 256 * (c0 >> 7) + 128 * hh + (c0 & 127);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(acc[j]) * inv_l, __uint_as_float(acc[j + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(acc[j + 2]) * inv_l, __uint_as_float(acc[j + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(acc[j + 4]) * inv_l, __uint_as_float(acc[j + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(acc[j + 6]) * inv_l, __uint_as_float(acc[j + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + dv0 + j) = v;
        }
      }
    }
    if (hh == 0 && head < p.h) {
      float v = -INFINITY;
      if (l_tot > 0.0f) {
        const float l2 = m_run + log2f(l_tot);
        v = p.lse_base2 ? l2 : l2 * 0.6931471805599453f;
      }
      p.lse[static_cast<long long>(token) * p.lse_st + head] = v;
    }
    tc_fence_before();
  } else if (warp == 4) {
    // ---------------------------------------------------------------- MMA issuer (even CTA, one thread)
    if (cta == 0 && lane == 0) {
      constexpr uint32_t kIdescQK = umma_idesc(kFmtBF16, 128, kNT, 0, 0);
      constexpr uint32_t kIdescPV = umma_idesc(kFmtBF16, 128, 256, 0, 1);
      const uint32_t s_full_a[2][2] = {{mapa_shared(smem_u32(&misc->s_full[0]), 0), mapa_shared(smem_u32(&misc->s_full[0]), 1)},
                                       {mapa_shared(smem_u32(&misc->s_full[1]), 0), mapa_shared(smem_u32(&misc->s_full[1]), 1)}};
      const uint32_t pv_done_a[2][2] = {{mapa_shared(smem_u32(&misc->pv_done[0]), 0), mapa_shared(smem_u32(&misc->pv_done[0]), 1)},
                                        {mapa_shared(smem_u32(&misc->pv_done[1]), 0), mapa_shared(smem_u32(&misc->pv_done[1]), 1)}};
      auto issue_qk = [&](int i) {
        const int b = i & 1;
        mbar_wait(smem_u32(&misc->k_full[b]), (i >> 1) & 1u, abort_flag);
        tc_fence_after();
#pragma unroll 1
        for (int cc = 0; cc < kNChunk; ++cc) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = smem_desc_sw128(q_s + cc * kQBlock + k * 32, 16, 1024);
            const uint64_t bd = smem_desc_sw128(k_s + b * kKStage + cc * kKBlock + k * 32, 16, 1024);
            umma_f16_ss_pair(tmem + kColS + b * 32, ad, bd, kIdescQK, (cc | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(s_full_a[b][0]);
        umma_commit_pair(s_full_a[b][1]);
      };
      auto issue_pv = [&](int i) {
        const int b = i & 1;
        mbar_wait(smem_u32(&misc->v_full[b]), (i >> 1) & 1u, abort_flag);
        mbar_wait(smem_u32(&misc->p_full[b]), (i >> 1) & 1u, abort_flag);
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = smem_desc_sw128(p_s + b * kPBytes + k * 32, 16, 1024);
            const uint64_t bd = smem_desc_sw128(v_s + b * kVStage + half * 2 * kVBlock + k * 2048, kVBlock, 1024);
            umma_f16_ss_pair(tmem + kColO + half * 128, ad, bd, kIdescPV, (i | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit_pair(pv_done_a[b][0]);
        umma_commit_pair(pv_done_a[b][1]);
      };
      if (n_tiles > 0) issue_qk(0);
      for (int i = 0; i < n_tiles; ++i) {
        if (i + 1 < n_tiles) issue_qk(i + 1);     // overlaps the softmax of tile i
        issue_pv(i);
      }
    }
  } else if (warp < 9) {
    // ---------------------------------------------------------------- K producers (warps 5-8, 128 threads)
    // A warp copies whole rows: lanes cover consecutive 16-byte chunks of one gathered row (72 per row,
    // three warp-wide cp.async), so no per-chunk index arithmetic and full 32-byte sectors.
    const int pt = tid - 160;                        // 0..127
    const int pw = warp - 5;                         // 0..3: rows pw*8 .. pw*8+7 of this CTA's 32
    const uint32_t k_full0 = mapa_shared(smem_u32(&misc->k_full[0]), 0);
    const uint32_t k_full1 = mapa_shared(smem_u32(&misc->k_full[1]), 0);
    int idx_next = (pt < kNT && pt < p.topk) ? idx_row[pt] : -1;   // index of tile 0, slot pt
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      const int logical = idx_next;
      {
        const int jn = (i + 1) * kNT + pt;
        idx_next = (pt < kNT && i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
      }
      // K stage b was last read by Q.K^T of tile i-2
      if (i >= 2) mbar_wait(smem_u32(&misc->s_full[b]), ((i - 2) >> 1) & 1u, abort_flag);
      if (pt < kNT) {
        const bool ok = logical >= 0 && logical < p.s_kv;
        if (logical >= p.s_kv) misc->bad_index = 1;
        const uint32_t m = __ballot_sync(0xffffffffu, ok);
        if (lane == 0) misc->valid_mask[i & 3][pt >> 5] = m;
        if ((pt >> 5) == cta) misc->k_rows[b][pt & 31] = ok ? logical : 0;
      }
      named_bar_sync(3, 128);
      const uint32_t stage = k_s + b * kKStage;
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        const int r = pw * 8 + rr;
        const __nv_bfloat16* src = p.kv + static_cast<long long>(misc->k_rows[b][r]) * p.kv_sr;
        const uint32_t drow = stage + r * 128;
#pragma unroll
        for (int part = 0; part < 3; ++part) {
          const int ch = part * 32 + lane;
          if (ch < kDqk / 8)
            cp_async16(drow + (ch >> 3) * kKBlock + (((ch & 7) ^ (r & 7)) << 4), src + ch * 8);
        }
      }
      cp_async_commit();
      if (i >= 1) {
        // tile i-1 has landed (at most the group just committed is pending)
        cp_async_wait_group1();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(((i - 1) & 1) ? k_full1 : k_full0);
      }
    }
    if (n_tiles > 0) {
      cp_async_wait_group0();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(((n_tiles - 1) & 1) ? k_full1 : k_full0);
    }
  } else {
    // ---------------------------------------------------------------- V producers (warps 9-12, 128 threads)
    // One warp-wide cp.async per gathered row: the 32 lanes cover this CTA's four 64-column blocks
    // (two 256-byte runs of the latent row).
    const int pt = tid - 288;                        // 0..127
    const int pw = warp - 9;                         // rows pw*16 .. pw*16+15
    const uint32_t v_full0 = mapa_shared(smem_u32(&misc->v_full[0]), 0);
    const uint32_t v_full1 = mapa_shared(smem_u32(&misc->v_full[1]), 0);
    const int blk = lane >> 3;                       // block inside the V stage
    const int c16 = lane & 7;
    const int src_off = ((blk >> 1) * 4 + 2 * cta + (blk & 1)) * 64 + c16 * 8;   // element offset in the row
    int idx_next = (pt < kNT && pt < p.topk) ? idx_row[pt] : -1;
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      const int logical = idx_next;
      {
        const int jn = (i + 1) * kNT + pt;
        idx_next = (pt < kNT && i + 1 < n_tiles && jn < p.topk) ? idx_row[jn] : -1;
      }
      // V stage b was last read by P.V of tile i-2
      if (i >= 2) mbar_wait(smem_u32(&misc->pv_done[b]), ((i - 2) >> 1) & 1u, abort_flag);
      if (pt < kNT) misc->v_rows[b][pt] = (logical >= 0 && logical < p.s_kv) ? logical : 0;
      named_bar_sync(4, 128);
      const uint32_t stage = v_s + b * kVStage + blk * kVBlock;
#pragma unroll
      for (int rr = 0; rr < 16; ++rr) {
        const int r = pw * 16 + rr;
        cp_async16(stage + r * 128 + ((c16 ^ (r & 7)) << 4),
                   p.kv + static_cast<long long>(misc->v_rows[b][r]) * p.kv_sr + src_off);
      }
      cp_async_commit();
      if (i >= 1) {
        cp_async_wait_group1();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(((i - 1) & 1) ? v_full1 : v_full0);
      }
    }
    if (n_tiles > 0) {
      cp_async_wait_group0();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(((n_tiles - 1) & 1) ? v_full1 : v_full0);
    }
  }

  __syncthreads();
  cluster_sync_all();            // nobody leaves while the peer may still signal or read this CTA
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, kTmemCols);
  }
  if (tid == 0 && p.status != nullptr) {
    if (misc->abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
    else if (misc->bad_index) atomicCAS(p.status, 0, FTB_ERR_BAD_INDEX);
  }
}

}  // namespace mla2

// Launches the CTA-pair kernel; arguments were validated by the caller.
int launch_sparse_mla_pair(const ftb_sparse_mla_args* a, cudaStream_t st) {
  mla2::Params p;
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
  cudaError_t e = cudaFuncSetAttribute(mla2::sparse_mla_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla2::kSmemBytes);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla_pair)");
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(a->s_q) * 2u);
  cfg.blockDim = dim3(mla2::kThreads);
  cfg.dynamicSmemBytes = mla2::kSmemBytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, mla2::sparse_mla_pair_kernel, p);
  return check_cuda(e, "sparse_mla_pair launch");
}

}  // namespace ftb
