// Top-k sparse MLA forward for sm_100a: gather latent-KV rows by index into 128B-swizzled shared
// memory, S = Q.K^T and O += P.V on tcgen05 tensor cores with TMEM accumulators, online softmax
// in registers (one thread per head row).
//
// Work decomposition: one CTA per (query token, half of the 512 output columns).  TMEM holds
// 128 lanes x 512 fp32 columns per SM; a full O tile [128 heads x 512] would fill it, leaving no
// room for S, so each CTA owns O[128 x 256] (256 columns) plus S[128 x 64] (64 columns).
//
// Shared memory (1024-byte aligned, 128B swizzle = 16-byte chunk index XOR (row & 7)):
//   Q   : 9 column blocks (64 bf16 = 128 B wide) x 128 head rows x 128 B  = 147456 B
//   KV  : 9 column blocks x 64 gathered rows x 128 B                       =  73728 B
//   The same KV tile is the K-major B operand of Q.K^T (all 9 blocks) and the MN-major B
//   operand of P.V (the 4 blocks of this CTA's output half): the latent row is fetched once.
//   P   : 128 x 64 bf16 (16 KB), written over two KV column blocks that are dead once Q.K^T of
//         the tile has finished (the rope block and a block of the other output half).
#include <cuda_fp8.h>

#include "sm100.cuh"
#include "../../include/flagtree_b200.h"

namespace ftb {

constexpr int kDqk = 576;
constexpr int kDv = 512;
constexpr int kNChunk = kDqk / 64;          // 9 column blocks of 64 bf16
constexpr int kHeadsPerCta = 128;           // MMA M
constexpr int kBN = 64;                     // gathered rows per tile (MMA N of Q.K^T, K of P.V)
constexpr int kDvHalf = 256;                // output columns per CTA
constexpr int kQBlockBytes = kHeadsPerCta * 128;   // 16384
constexpr int kQBytes = kNChunk * kQBlockBytes;    // 147456
constexpr int kKvBlockBytes = kBN * 128;           // 8192
constexpr int kKvBytes = kNChunk * kKvBlockBytes;  // 73728
constexpr int kMiscBytes = 1024;
constexpr int kSmemBytes = kQBytes + kKvBytes + kMiscBytes + 1024;  // + alignment slack
constexpr int kThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemColO = 0;
constexpr uint32_t kTmemColS = 256;

struct MlaParams {
  const __nv_bfloat16* q;
  const void* kv;
  const int32_t* indices;
  __nv_bfloat16* out;
  float* lse;
  int s_q, h, s_kv, topk;
  long long q_st, q_sh, kv_sr, idx_st, out_st, out_sh, lse_st;
  float scale_log2;          // sm_scale * log2(e)
  int lse_base2;
  int* status;
  float* dbg_scores;
  const float* kv_scale;
  const int32_t* block_table;
  const int32_t* context_lens;
  int page_size, q_per_seq;
  long long bt_stride;
  // split over the top-k axis: partial results go to scratch and a second kernel merges them
  int n_splits;
  float* part_out;   // fp32 [s_q, n_splits, h, 512], each split normalised by its own sum
  float* part_lse;   // fp32 [s_q, n_splits, h], log2-domain log-sum-exp of the split (-inf = empty)
};

struct MiscSmem {
  unsigned long long bar_s;     // Q.K^T of the tile finished
  unsigned long long bar_o;     // P.V of the tile finished
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  uint32_t valid_mask[2];
  int bad_index;
  int rows[kBN];                // physical row of each tile column (0 when masked)
  float row_scale[kBN];         // per-row dequantisation scale (FP8 form)
};

__device__ __forceinline__ int resolve_row(const MlaParams& p, int token, int logical, bool& ok, float& scale, bool& bad) {
  // Returns the physical row for a top-k entry; ok = false for padding (-1, or at / past the context length);
  // bad = true for an entry that is neither padding nor a row of the cache (never dereferenced).
  scale = 1.0f;
  ok = false;
  bad = false;
  if (logical < 0) { bad = logical < -1; return 0; }
  if (p.block_table == nullptr) {
    ok = logical < p.s_kv;
    bad = !ok;
    return ok ? logical : 0;
  }
  const int seq = token / p.q_per_seq;
  if (logical >= p.context_lens[seq]) return 0;
  const int slot = logical / p.page_size;
  if (slot >= p.bt_stride) { bad = true; return 0; }      // a context length longer than the table's row
  const int page = p.block_table[seq * p.bt_stride + slot];
  const int row = page * p.page_size + logical % p.page_size;
  ok = page >= 0 && row >= 0 && row < p.s_kv;
  bad = !ok;
  if (ok && p.kv_scale != nullptr) scale = p.kv_scale[page];
  return ok ? row : 0;
}

// Paged FP8 form, first pass of the two-pass path: one warp per selected row.  The row is resolved through
// the page table, its 576 e4m3 values are converted to bf16 times the page scale (the same arithmetic as
// the gather of the one-pass kernel below) and written to row r = token * topk + j of a compact bf16 table;
// `out_idx[r]` is r, or -1 for padding and for positions at or past the context length.  The bf16 kernels
// then run on the compact table with these indices.
__global__ void __launch_bounds__(256) mla_dequant_rows_kernel(const MlaParams p, __nv_bfloat16* table, int32_t* out_idx) {
  const int lane = threadIdx.x & 31;
  const long long n_rows = static_cast<long long>(p.s_q) * p.topk;
  const uint8_t* kvp = reinterpret_cast<const uint8_t*>(p.kv);
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < n_rows;
       r += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int token = static_cast<int>(r / p.topk);
    const int j = static_cast<int>(r - static_cast<long long>(token) * p.topk);
    const int logical = p.indices[static_cast<long long>(token) * p.idx_st + j];
    bool ok, bad;
    float sc;
    const int row = resolve_row(p, token, logical, ok, sc, bad);
    if (bad && lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, FTB_ERR_BAD_INDEX);
    if (lane == 0) out_idx[r] = ok ? static_cast<int32_t>(r) : -1;
    if (!ok) {
      // the attention kernel fetches table row 0 for every masked entry (and multiplies it by zero): that row
      // must hold finite numbers even when its own entry is masked
      if (r == 0) {
        uint4* z = reinterpret_cast<uint4*>(table);
        for (int c16 = lane; c16 < kDqk * 2 / 16; c16 += 32) z[c16] = make_uint4(0, 0, 0, 0);
      }
      continue;
    }
    const uint8_t* src = kvp + static_cast<long long>(row) * p.kv_sr;
    uint32_t* dst = reinterpret_cast<uint32_t*>(table + r * kDqk);
    // 36 chunks of 16 bytes: every lane one, lanes 0-3 a second one
    for (int c16 = lane; c16 < kDqk / 16; c16 += 32) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c16 * 16);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_fp8x2_storage_t lo = static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu);
        const __nv_fp8x2_storage_t hi = static_cast<__nv_fp8x2_storage_t>(w[i] >> 16);
        const __half2_raw hlo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3);
        const __half2_raw hhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
        const float2 flo = __half22float2(*reinterpret_cast<const __half2*>(&hlo));
        const float2 fhi = __half22float2(*reinterpret_cast<const __half2*>(&hhi));
        o[2 * i] = pack_bf16x2(flo.x * sc, flo.y * sc);
        o[2 * i + 1] = pack_bf16x2(fhi.x * sc, fhi.y * sc);
      }
      reinterpret_cast<uint4*>(dst)[c16 * 2] = make_uint4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<uint4*>(dst)[c16 * 2 + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

template <bool kFp8>
__global__ void __launch_bounds__(kThreads, 1) sparse_mla_fwd_kernel(const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  const uint32_t q_s = base;
  const uint32_t kv_s = base + kQBytes;
  MiscSmem* misc = reinterpret_cast<MiscSmem*>(sm + kQBytes + kKvBytes);
  const uint32_t bar_s = smem_u32(&misc->bar_s);
  const uint32_t bar_o = smem_u32(&misc->bar_o);
  volatile int* abort_flag = &misc->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int hv = blockIdx.x & 1;
  const int split = (blockIdx.x >> 1) % p.n_splits;
  const int token = (blockIdx.x >> 1) / p.n_splits;
  // P overwrites KV column blocks that this CTA's P.V does not read.
  const uint32_t p_s = kv_s + (hv == 0 ? 7 : 0) * kKvBlockBytes;
  const uint32_t v_s = kv_s + (hv * 4) * kKvBlockBytes;

  if (tid == 0) {
    misc->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    misc->n_scan = 0;
    misc->bad_index = 0;
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (misc->abort_flag) return;   // an earlier CTA of this launch already failed: do nothing

  if (warp == 0) {
    tmem_alloc(smem_u32(&misc->tmem_base), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }

  // Number of leading top-k slots that must be visited (last valid slot + 1).
  {
    int local = 0;
    const int32_t* idx_row = p.indices + static_cast<long long>(token) * p.idx_st;
    for (int j = tid; j < p.topk; j += kThreads) {
      const int v = idx_row[j];
      if (v >= 0) local = j + 1;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = max(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0 && local > 0) atomicMax(&misc->n_scan, local);
  }

  // Q tile -> shared memory (rows >= h are zero).
  {
    const __nv_bfloat16* q_tok = p.q + static_cast<long long>(token) * p.q_st;
    for (int c = tid; c < kHeadsPerCta * (kDqk / 8); c += kThreads) {
      const int r = c / (kDqk / 8);
      const int ch = c - r * (kDqk / 8);
      const uint32_t dst = q_s + (ch >> 3) * kQBlockBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
      if (r < p.h) {
        cp_async16(dst, q_tok + static_cast<long long>(r) * p.q_sh + ch * 8);
      } else {
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
      }
    }
    cp_async_commit();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc->tmem_base;
  const int n_tiles = (misc->n_scan + kBN - 1) / kBN;

  constexpr uint32_t kIdescQK = umma_idesc(kFmtBF16, 128, kBN, 0, 0);
  constexpr uint32_t kIdescPV = umma_idesc(kFmtBF16, 128, kDvHalf, 0, 1);

  float m_run = -INFINITY;   // running max in the log2 domain (score * scale_log2)
  float l_run = 0.0f;        // running sum of 2^(s - m_run)

  // this CTA's share of the tiles (all of them unless the top-k axis is split)
  const int tiles_per_split = (n_tiles + p.n_splits - 1) / p.n_splits;
  const int t0 = split * tiles_per_split;
  const int t1 = min(n_tiles, t0 + tiles_per_split);

  for (int tile = t0; tile < t1; ++tile) {
    const uint32_t parity = (tile - t0) & 1;
    // ---- indices of this tile
    if (tid < kBN) {
      const int j = tile * kBN + tid;
      int logical = -1;
      if (j < p.topk) logical = p.indices[static_cast<long long>(token) * p.idx_st + j];
      bool ok, bad;
      float sc;
      const int row = resolve_row(p, token, logical, ok, sc, bad);
      if (bad) misc->bad_index = 1;
      misc->rows[tid] = row;
      misc->row_scale[tid] = sc;
      const uint32_t m = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) misc->valid_mask[warp] = m;
    }
    __syncthreads();

    // ---- gather the tile's rows into the swizzled KV tile
    if constexpr (!kFp8) {
      const __nv_bfloat16* kvp = reinterpret_cast<const __nv_bfloat16*>(p.kv);
      for (int c = tid; c < kBN * (kDqk / 8); c += kThreads) {
        const int r = c / (kDqk / 8);
        const int ch = c - r * (kDqk / 8);
        const uint32_t dst = kv_s + (ch >> 3) * kKvBlockBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
        cp_async16(dst, kvp + static_cast<long long>(misc->rows[r]) * p.kv_sr + ch * 8);
      }
      cp_async_commit();
    } else {
      // e4m3 rows: 16 bytes = 16 elements -> two 16-byte bf16 chunks, scaled by the page scale.
      const uint8_t* kvp = reinterpret_cast<const uint8_t*>(p.kv);
      for (int c = tid; c < kBN * (kDqk / 16); c += kThreads) {
        const int r = c / (kDqk / 16);
        const int c16 = c - r * (kDqk / 16);
        const uint4 raw = *reinterpret_cast<const uint4*>(kvp + static_cast<long long>(misc->rows[r]) * p.kv_sr + c16 * 16);
        const float sc = misc->row_scale[r];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_fp8x2_storage_t lo = static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu);
          const __nv_fp8x2_storage_t hi = static_cast<__nv_fp8x2_storage_t>(w[i] >> 16);
          const __half2_raw hlo = __nv_cvt_fp8x2_to_halfraw2(lo, __NV_E4M3);
          const __half2_raw hhi = __nv_cvt_fp8x2_to_halfraw2(hi, __NV_E4M3);
          const float2 flo = __half22float2(*reinterpret_cast<const __half2*>(&hlo));
          const float2 fhi = __half22float2(*reinterpret_cast<const __half2*>(&hhi));
          o[2 * i] = pack_bf16x2(flo.x * sc, flo.y * sc);
          o[2 * i + 1] = pack_bf16x2(fhi.x * sc, fhi.y * sc);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int ch = c16 * 2 + half;
          const uint32_t dst = kv_s + (ch >> 3) * kKvBlockBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[4 * half]), "r"(o[4 * half + 1]),
                       "r"(o[4 * half + 2]), "r"(o[4 * half + 3])
                       : "memory");
        }
      }
    }
    cp_async_wait_all();
    fence_proxy_async_smem();
    __syncthreads();

    // ---- S = Q.K^T  (36 MMAs of 128 x 64 x 16)
    if (tid == 0) {
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < kNChunk; ++cc) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t ad = smem_desc_sw128(q_s + cc * kQBlockBytes + k * 32, 16, 1024);
          const uint64_t bd = smem_desc_sw128(kv_s + cc * kKvBlockBytes + k * 32, 16, 1024);
          umma_f16_ss(tmem + kTmemColS, ad, bd, kIdescQK, (cc | k) != 0 ? 1u : 0u);
        }
      }
      umma_commit(bar_s);
    }

    // ---- softmax on the 128 head rows (warps 0-3: thread == TMEM lane == head)
    if (warp < 4) {
      mbar_wait(bar_s, parity, abort_flag);
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(tmem_addr(tmem, warp * 32, kTmemColS), sr[0]);
      tmem_ld32(tmem_addr(tmem, warp * 32, kTmemColS + 32), sr[1]);
      tmem_wait_ld();
      if (p.dbg_scores != nullptr) {
        const int topk_pad = ((p.topk + kBN - 1) / kBN) * kBN;
        float* d = p.dbg_scores + (static_cast<long long>(token) * 128 + tid) * topk_pad + tile * kBN;
        if (hv == 0) {
#pragma unroll
          for (int j = 0; j < 64; ++j) d[j] = __uint_as_float(sr[j >> 5][j & 31]);
        }
      }
      const uint32_t vm0 = misc->valid_mask[0], vm1 = misc->valid_mask[1];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if ((vm0 >> j) & 1u) mx = fmaxf(mx, __uint_as_float(sr[0][j]));
        if ((vm1 >> j) & 1u) mx = fmaxf(mx, __uint_as_float(sr[1][j]));
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_use);
      float psum = 0.0f;
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        // columns j, j+1 of the first half and of the second half
        float a0 = ((vm0 >> j) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[0][j]), p.scale_log2, -m_use)) : 0.0f;
        float a1 = ((vm0 >> (j + 1)) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[0][j + 1]), p.scale_log2, -m_use)) : 0.0f;
        float b0 = ((vm1 >> j) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[1][j]), p.scale_log2, -m_use)) : 0.0f;
        float b1 = ((vm1 >> (j + 1)) & 1u) ? fast_exp2(fmaf(__uint_as_float(sr[1][j + 1]), p.scale_log2, -m_use)) : 0.0f;
        psum += (a0 + a1) + (b0 + b1);
        pk[j >> 1] = pack_bf16x2(a0, a1);
        pk[16 + (j >> 1)] = pack_bf16x2(b0, b1);
      }
      l_run = l_run * alpha + psum;
      m_run = m_new;
      // P row -> shared memory (K-major, 128 B per row, swizzled)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t dst = p_s + tid * 128 + ((c ^ (tid & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                     "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                     : "memory");
      }
      // Rescale the running O when the row max moved (whole warp takes part: TMEM ops are collective).
      const bool need = (tile > t0) && (alpha != 1.0f);
      if (__any_sync(0xffffffffu, need)) {
        const float a = (tile > t0) ? alpha : 1.0f;
#pragma unroll 1
        for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
          uint32_t orow[32];
          tmem_ld32(tmem_addr(tmem, warp * 32, kTmemColO + c0), orow);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) orow[j] = __float_as_uint(__uint_as_float(orow[j]) * a);
          tmem_st32(tmem_addr(tmem, warp * 32, kTmemColO + c0), orow);
        }
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before();
    }
    __syncthreads();

    // ---- O += P.V  (4 MMAs of 128 x 256 x 16; V is the MN-major view of the gathered tile)
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t ad = smem_desc_sw128(p_s + k * 32, 16, 1024);
        const uint64_t bd = smem_desc_sw128(v_s + k * 2048, kKvBlockBytes, 1024);
        umma_f16_ss(tmem + kTmemColO, ad, bd, kIdescPV, (tile != t0 || k != 0) ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
    // The tile's shared memory and O are reused by the next iteration: wait for the MMAs.
    mbar_wait(bar_o, parity, abort_flag);
    tc_fence_after();
  }

  // ---- epilogue: O / l -> bf16 and LSE, or the fp32 partial of this split
  if (warp < 4) {
    const int head = tid;
    const float inv_l = (l_run > 0.0f) ? 1.0f / l_run : 0.0f;
    __nv_bfloat16* orow = p.out + static_cast<long long>(token) * p.out_st + static_cast<long long>(head) * p.out_sh + hv * kDvHalf;
    float* prow = nullptr;
    if (p.n_splits > 1)
      prow = p.part_out + ((static_cast<long long>(token) * p.n_splits + split) * p.h + head) * 512 + hv * kDvHalf;
#pragma unroll 1
    for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
      uint32_t acc[32];
      if (t1 > t0) {
        tmem_ld32(tmem_addr(tmem, warp * 32, kTmemColO + c0), acc);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
      }
      if (head < p.h) {
        if (prow != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v;
            v.x = __uint_as_float(acc[j]) * inv_l;
            v.y = __uint_as_float(acc[j + 1]) * inv_l;
            v.z = __uint_as_float(acc[j + 2]) * inv_l;
            v.w = __uint_as_float(acc[j + 3]) * inv_l;
            *reinterpret_cast<float4*>(prow + c0 + j) = v;
          }
        } else {
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
    }
    if (hv == 0 && head < p.h) {
      const float l2 = (l_run > 0.0f) ? m_run + log2f(l_run) : -INFINITY;
      if (p.n_splits > 1) {
        p.part_lse[(static_cast<long long>(token) * p.n_splits + split) * p.h + head] = l2;
      } else {
        p.lse[static_cast<long long>(token) * p.lse_st + head] = (p.lse_base2 || l2 == -INFINITY) ? l2 : l2 * 0.6931471805599453f;
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && p.status != nullptr) {
    if (misc->abort_flag) atomicCAS(p.status, 0, FTB_ERR_TIMEOUT);
    else if (misc->bad_index) atomicCAS(p.status, 0, FTB_ERR_BAD_INDEX);
  }
}


// Merge of the per-split partial results (the role of the reference's _fwd_kernel_stage2,
// third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py:426-477): weights 2^(lse_k - max),
// out = sum w_k out_k / sum w_k, and the merged LSE, which the reference does not store.
// One warp per (token, head); lane i owns output columns [16 i, 16 i + 16).
__global__ void __launch_bounds__(256) sparse_mla_merge_kernel(const float* __restrict__ part_out,
                                                               const float* __restrict__ part_lse, __nv_bfloat16* out,
                                                               float* lse, int s_q, int h, int n_splits, long long out_st,
                                                               long long out_sh, long long lse_st, int lse_base2) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= s_q * h) return;
  const int token = w / h, head = w - token * h;
  float mx = -INFINITY;
  for (int k = 0; k < n_splits; ++k) mx = fmaxf(mx, part_lse[(static_cast<long long>(token) * n_splits + k) * h + head]);
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  float wsum = 0.0f;
  if (mx != -INFINITY) {
    for (int k = 0; k < n_splits; ++k) {
      const long long row = (static_cast<long long>(token) * n_splits + k) * h + head;
      const float l2 = part_lse[row];
      if (l2 == -INFINITY) continue;
      const float wk = fast_exp2(l2 - mx);
      wsum += wk;
      const float4* src = reinterpret_cast<const float4*>(part_out + row * 512 + lane * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 v = src[j];
        acc[4 * j] += wk * v.x; acc[4 * j + 1] += wk * v.y; acc[4 * j + 2] += wk * v.z; acc[4 * j + 3] += wk * v.w;
      }
    }
  }
  const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
  uint4 o[2];
  uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j) ow[j] = pack_bf16x2(acc[2 * j] * inv, acc[2 * j + 1] * inv);
  uint4* dst = reinterpret_cast<uint4*>(out + token * out_st + head * out_sh + lane * 16);
  dst[0] = o[0];
  dst[1] = o[1];
  if (lane == 0) {
    const float l2 = wsum > 0.0f ? mx + log2f(wsum) : -INFINITY;
    lse[token * lse_st + head] = (lse_base2 || l2 == -INFINITY) ? l2 : l2 * 0.6931471805599453f;
  }
}


// The same merge for partial results that come from outside the library: the outputs and log-sum-exps of
// several sparse-MLA forwards over disjoint parts of the key/value rows (a long context sharded over GPUs, or
// a caller's own split of the top-k list).  part k of (token, head): `part_out + k * ps + token * ts + head * hs`
// (T = bf16, what ftb_sparse_mla_fwd writes, or fp32), its log-sum-exp `part_lse + k * lps + token * lts + head`
// (natural log, or base 2 when lse_base2; -inf = the part saw no valid row).  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256) sparse_mla_merge_parts_kernel(const T* __restrict__ part_out, const float* __restrict__ part_lse,
                                                                     __nv_bfloat16* out, float* lse, int s_q, int h, int n_parts,
                                                                     long long ps, long long ts, long long hs, long long lps,
                                                                     long long lts, long long out_st, long long out_sh,
                                                                     long long lse_st, int lse_base2) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= s_q * h) return;
  const int token = w / h, head = w - token * h;
  const float to2 = lse_base2 ? 1.0f : 1.4426950408889634f;      // natural log -> base 2
  const float* lrow = part_lse + static_cast<long long>(token) * lts + head;
  float mx = -INFINITY;
  for (int k = 0; k < n_parts; ++k) mx = fmaxf(mx, lrow[k * lps] * to2);
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  float wsum = 0.0f;
  if (mx != -INFINITY) {
    for (int k = 0; k < n_parts; ++k) {
      const float l2 = lrow[k * lps] * to2;
      if (l2 == -INFINITY) continue;
      const float wk = exp2f(l2 - mx);
      wsum += wk;
      const T* src = part_out + k * ps + static_cast<long long>(token) * ts + static_cast<long long>(head) * hs + lane * 16;
      if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 v = reinterpret_cast<const float4*>(src)[j];
          acc[4 * j] += wk * v.x; acc[4 * j + 1] += wk * v.y; acc[4 * j + 2] += wk * v.z; acc[4 * j + 3] += wk * v.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint4 v = reinterpret_cast<const uint4*>(src)[j];
          const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[8 * j + 2 * e] += wk * __uint_as_float(u[e] << 16);
            acc[8 * j + 2 * e + 1] += wk * __uint_as_float(u[e] & 0xffff0000u);
          }
        }
      }
    }
  }
  const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
  uint4 o[2];
  uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j) ow[j] = pack_bf16x2(acc[2 * j] * inv, acc[2 * j + 1] * inv);
  uint4* dst = reinterpret_cast<uint4*>(out + token * out_st + head * out_sh + lane * 16);
  dst[0] = o[0];
  dst[1] = o[1];
  if (lane == 0) {
    const float l2 = wsum > 0.0f ? mx + log2f(wsum) : -INFINITY;
    lse[token * lse_st + head] = (lse_base2 || l2 == -INFINITY) ? l2 : l2 * 0.6931471805599453f;
  }
}

}  // namespace ftb

// --------------------------------------------------------------------------------- host side
#include <cstdio>
#include <cstring>

namespace ftb {
void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int launch_sparse_mla_ring(const ftb_sparse_mla_args* a, cudaStream_t st);
int launch_sparse_mla_few(const ftb_sparse_mla_args* a, cudaStream_t st);
}  // namespace ftb

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" FTB_API int ftb_sparse_mla_fwd(const ftb_sparse_mla_args* a, void* stream) {
  using namespace ftb;
  if (a == nullptr) { set_last_error("ftb_sparse_mla_fwd: args is NULL"); return FTB_ERR_INVALID; }
  if (a->s_q < 0 || a->h <= 0 || a->s_kv <= 0 || a->topk < 0) {
    set_last_error("ftb_sparse_mla_fwd: bad sizes s_q=%d h=%d s_kv=%d topk=%d", a->s_q, a->h, a->s_kv, a->topk);
    return FTB_ERR_INVALID;
  }
  if (a->s_q == 0) return FTB_OK;
  if (a->h > kHeadsPerCta) {
    set_last_error("ftb_sparse_mla_fwd: h=%d exceeds %d heads per launch", a->h, kHeadsPerCta);
    return FTB_ERR_UNSUPPORTED;
  }
  if (!a->q || !a->kv || !a->out || !a->lse || (a->topk > 0 && !a->indices)) {
    set_last_error("ftb_sparse_mla_fwd: null tensor pointer");
    return FTB_ERR_INVALID;
  }
  if (!aligned16(a->q) || !aligned16(a->kv) || !aligned16(a->out) || (a->q_stride_token % 8) || (a->q_stride_head % 8) ||
      (a->out_stride_token % 8) || (a->out_stride_head % 8)) {
    set_last_error("ftb_sparse_mla_fwd: q/kv/out must be 16-byte aligned with strides that are multiples of 8 elements");
    return FTB_ERR_INVALID;
  }
  if (a->kv_is_fp8) {
    if (a->kv_stride_row % 16) { set_last_error("ftb_sparse_mla_fwd: fp8 kv row stride must be a multiple of 16"); return FTB_ERR_INVALID; }
    if (!a->block_table || !a->context_lens || !a->kv_scale || a->page_size <= 0 || a->q_per_seq <= 0) {
      set_last_error("ftb_sparse_mla_fwd: paged fp8 form needs block_table, context_lens, kv_scale, page_size, q_per_seq");
      return FTB_ERR_INVALID;
    }
  } else if (a->kv_stride_row % 8) {
    set_last_error("ftb_sparse_mla_fwd: kv row stride must be a multiple of 8 elements");
    return FTB_ERR_INVALID;
  }
  // algo 0 = default = 5: persistent role-split CTA pairs (scores in one CTA, values in the other, Q in tensor
  // memory, one ring for K and Q filled by TMA row gathers); algo 1 = one CTA per (token, output half), which is
  // also the kernel of the FP8 paged form without a workspace, of the split form and of the diagnostic score tap;
  // algo 6 = paged FP8 form: dequantise the selected rows, then the persistent kernel; algo 2 = few heads (h <= 32):
  // one CTA per token, the gathered rows on the rows of the MMA.  Measured at h = 16 / 32 (2048 causal tokens,
  // topk 2048): 0.89 / 1.14 ms against 0.80 ms of the persistent pairs, so the default keeps the pairs: an MMA with
  // 16 columns costs what one with 128 costs (its time goes with the 128 rows of the A operand), so putting the
  // heads on the columns saves no tensor time, and this kernel does not overlap its gather with its products.
  if (a->algo_id != 0 && a->algo_id != 1 && a->algo_id != 2 && a->algo_id != 5 && a->algo_id != 6) {
    set_last_error("ftb_sparse_mla_fwd: unknown algo_id %d (0 = default, 1, 2, 5, 6)", a->algo_id);
    return FTB_ERR_INVALID;
  }
  if (a->sm_scale <= 0.0f) { set_last_error("ftb_sparse_mla_fwd: sm_scale must be positive"); return FTB_ERR_INVALID; }
  const bool plain = !a->kv_is_fp8 && a->dbg_scores == nullptr && a->n_splits <= 1;
  if (a->algo_id == 2 && (!plain || a->h > 32)) {
    set_last_error("ftb_sparse_mla_fwd: algo 2 serves the bf16 form without splits for at most 32 heads");
    return FTB_ERR_INVALID;
  }
  if (a->algo_id == 2) return launch_sparse_mla_few(a, reinterpret_cast<cudaStream_t>(stream));
  if (!a->kv_is_fp8 && a->dbg_scores == nullptr && a->n_splits <= 1 && (a->algo_id == 0 || a->algo_id == 5))
    return launch_sparse_mla_ring(a, reinterpret_cast<cudaStream_t>(stream));
  MlaParams p;
  memset(&p, 0, sizeof(p));
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.kv = a->kv;
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
  p.dbg_scores = a->dbg_scores;
  if (a->kv_is_fp8) {
    p.kv_scale = a->kv_scale; p.block_table = a->block_table; p.context_lens = a->context_lens;
    p.page_size = a->page_size; p.q_per_seq = a->q_per_seq; p.bt_stride = a->block_table_stride;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int n_splits = a->n_splits > 0 ? a->n_splits : 1;
  // Paged FP8 form with a workspace for the dequantised rows (algo 0 or 6, no split): convert the selected
  // rows once, then run the persistent bf16 kernel on the compact table.  Without such a workspace the
  // one-pass kernel below converts while it gathers.
  if (a->kv_is_fp8 && n_splits == 1 && a->dbg_scores == nullptr && (a->algo_id == 0 || a->algo_id == 6)) {
    const int64_t need = ftb_sparse_mla_dequant_workspace_bytes(a->s_q, a->topk);
    const bool have = a->workspace != nullptr && a->workspace_bytes >= need && need > 0 &&
                      (reinterpret_cast<uintptr_t>(a->workspace) & 15u) == 0 &&
                      static_cast<long long>(a->s_q) * a->topk < (1LL << 31);
    if (a->algo_id == 6 && !have) {
      set_last_error("ftb_sparse_mla_fwd: algo 6 needs a 16-byte aligned workspace of ftb_sparse_mla_dequant_workspace_bytes() bytes");
      return FTB_ERR_INVALID;
    }
    if (have) {
      p.topk = a->topk;
      __nv_bfloat16* table = reinterpret_cast<__nv_bfloat16*>(a->workspace);
      int32_t* idx2 = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(a->workspace) +
                                                static_cast<size_t>(a->s_q) * a->topk * kDqk * 2);
      const long long n_rows = static_cast<long long>(a->s_q) * a->topk;
      const unsigned blocks = static_cast<unsigned>(n_rows / 8 < 148 * 16 ? (n_rows + 7) / 8 : 148 * 16);
      mla_dequant_rows_kernel<<<blocks, 256, 0, st>>>(p, table, idx2);
      int rc0 = check_cuda(cudaGetLastError(), "mla_dequant_rows launch");
      if (rc0 != FTB_OK) return rc0;
      ftb_sparse_mla_args b = *a;
      b.kv = table;
      b.kv_is_fp8 = 0;
      b.kv_scale = nullptr; b.block_table = nullptr; b.context_lens = nullptr;
      b.s_kv = static_cast<int32_t>(n_rows);
      b.kv_stride_row = kDqk;
      b.indices = idx2;
      b.idx_stride_token = a->topk;
      b.algo_id = 5;
      b.workspace = nullptr; b.workspace_bytes = 0; b.n_splits = 0;
      return launch_sparse_mla_ring(&b, st);
    }
  }
  if (n_splits > 1) {
    if (a->workspace == nullptr || a->workspace_bytes < ftb_sparse_mla_workspace_bytes(a->s_q, a->h, n_splits)) {
      set_last_error("ftb_sparse_mla_fwd: n_splits=%d needs a workspace of ftb_sparse_mla_workspace_bytes() bytes", n_splits);
      return FTB_ERR_INVALID;
    }
    p.part_out = reinterpret_cast<float*>(a->workspace);
    p.part_lse = p.part_out + static_cast<size_t>(a->s_q) * n_splits * a->h * 512;
  }
  p.n_splits = n_splits;
  const dim3 grid(static_cast<unsigned>(a->s_q) * 2u * static_cast<unsigned>(n_splits)), block(kThreads);
  cudaError_t e;
  if (a->kv_is_fp8) {
    e = cudaFuncSetAttribute(sparse_mla_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla fp8)");
    sparse_mla_fwd_kernel<true><<<grid, block, kSmemBytes, st>>>(p);
  } else {
    e = cudaFuncSetAttribute(sparse_mla_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla)");
    sparse_mla_fwd_kernel<false><<<grid, block, kSmemBytes, st>>>(p);
  }
  int rc = check_cuda(cudaGetLastError(), "sparse_mla_fwd launch");
  if (rc != FTB_OK || n_splits == 1) return rc;
  const int warps = a->s_q * a->h;
  sparse_mla_merge_kernel<<<(warps * 32 + 255) / 256, 256, 0, st>>>(p.part_out, p.part_lse, p.out, p.lse, a->s_q, a->h, n_splits,
                                                                    p.out_st, p.out_sh, p.lse_st, p.lse_base2);
  return check_cuda(cudaGetLastError(), "sparse_mla_merge launch");
}

extern "C" FTB_API int64_t ftb_sparse_mla_dequant_workspace_bytes(int32_t s_q, int32_t topk) {
  if (s_q <= 0 || topk <= 0) return 0;
  return static_cast<int64_t>(s_q) * topk * (576 * 2 + 4);
}

extern "C" FTB_API int64_t ftb_sparse_mla_workspace_bytes(int32_t s_q, int32_t h, int32_t n_splits) {
  if (n_splits <= 1 || s_q <= 0 || h <= 0) return 0;
  return static_cast<int64_t>(s_q) * n_splits * h * (512 + 1) * 4;
}


// ---------------------------------------------------------------------------------------------
// Entry point for callers that may not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a serving engine that has
// handed all device memory to its own pool, inside a plugin sandbox whose allocator hooks reject
// foreign allocations, or on a path that must not touch the allocator because a synchronising
// allocation would stall other streams.  For them the scratch of the split sparse-MLA forward (the
// per-split partial outputs and their log-sum-exps) lives in a fixed array inside the library image.
// The array costs FTB_MLA_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library,
// from load until the process exits, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------------------------
#define FTB_MLA_STATIC_SCRATCH_BYTES (32ll << 20)
static __device__ __align__(256) unsigned char g_mla_static_scratch[FTB_MLA_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the runtime, not an address a kernel can use;
// the device address is looked up once per device, with that device current.
static void* g_mla_static_scratch_addr[64] = {nullptr};

extern "C" FTB_API int64_t ftb_sparse_mla_static_scratch_bytes(void) { return FTB_MLA_STATIC_SCRATCH_BYTES; }

extern "C" FTB_API int ftb_sparse_mla_fwd_static_scratch(const ftb_sparse_mla_args* a, void* stream) {
  using namespace ftb;
  if (a == nullptr) { set_last_error("ftb_sparse_mla_fwd_static_scratch: args is NULL"); return FTB_ERR_INVALID; }
  const int64_t need = ftb_sparse_mla_workspace_bytes(a->s_q, a->h, a->n_splits);
  if (need > FTB_MLA_STATIC_SCRATCH_BYTES) {
    set_last_error("ftb_sparse_mla_fwd_static_scratch: s_q=%d x n_splits=%d x h=%d needs %lld bytes of scratch, the built-in "
                   "array holds %lld; use fewer splits or ftb_sparse_mla_fwd with a caller-provided workspace",
                   a->s_q, a->n_splits, a->h, static_cast<long long>(need), static_cast<long long>(FTB_MLA_STATIC_SCRATCH_BYTES));
    return FTB_ERR_INVALID;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return check_cuda(e, "ftb_sparse_mla_fwd_static_scratch: cudaGetDevice");
  if (dev < 0 || dev >= 64) { set_last_error("ftb_sparse_mla_fwd_static_scratch: device ordinal %d out of range", dev); return FTB_ERR_INVALID; }
  if (g_mla_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_mla_static_scratch);
    if (e != cudaSuccess) return check_cuda(e, "ftb_sparse_mla_fwd_static_scratch: cudaGetSymbolAddress");
    g_mla_static_scratch_addr[dev] = ptr;
  }
  ftb_sparse_mla_args b = *a;
  if (a->n_splits > 1) {
    b.workspace = g_mla_static_scratch_addr[dev];
    b.workspace_bytes = FTB_MLA_STATIC_SCRATCH_BYTES;
  } else {   // no split, no scratch (and no two-pass FP8 path through this entry)
    b.workspace = nullptr;
    b.workspace_bytes = 0;
  }
  return ftb_sparse_mla_fwd(&b, stream);
}


extern "C" FTB_API int ftb_sparse_mla_merge(const ftb_sparse_mla_merge_args* a, void* stream) {
  using namespace ftb;
  if (a == nullptr) { set_last_error("ftb_sparse_mla_merge: args is NULL"); return FTB_ERR_INVALID; }
  if (a->s_q < 0 || a->h <= 0 || a->n_parts <= 0) {
    set_last_error("ftb_sparse_mla_merge: bad sizes s_q=%d h=%d n_parts=%d", a->s_q, a->h, a->n_parts);
    return FTB_ERR_INVALID;
  }
  if (a->s_q == 0) return FTB_OK;
  if (!a->part_out || !a->part_lse || !a->out || !a->lse) { set_last_error("ftb_sparse_mla_merge: null pointer"); return FTB_ERR_INVALID; }
  if (a->part_is_fp32 != 0 && a->part_is_fp32 != 1) { set_last_error("ftb_sparse_mla_merge: part_is_fp32 must be 0 or 1"); return FTB_ERR_INVALID; }
  const int el = a->part_is_fp32 ? 4 : 8;      // elements per 16 bytes
  if (!aligned16(a->part_out) || !aligned16(a->out) || (a->part_stride_part % el) || (a->part_stride_token % el) ||
      (a->part_stride_head % el) || (a->out_stride_token % 8) || (a->out_stride_head % 8)) {
    set_last_error("ftb_sparse_mla_merge: part_out / out must be 16-byte aligned with strides that keep rows 16-byte aligned");
    return FTB_ERR_INVALID;
  }
  if (static_cast<long long>(a->s_q) * a->h > (1LL << 26)) { set_last_error("ftb_sparse_mla_merge: s_q * h too large for one launch"); return FTB_ERR_UNSUPPORTED; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int warps = a->s_q * a->h;
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(warps) * 32 + 255) / 256);
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a->out);
  if (a->part_is_fp32) {
    sparse_mla_merge_parts_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(a->part_out), a->part_lse, out, a->lse, a->s_q, a->h,
        a->n_parts, a->part_stride_part, a->part_stride_token, a->part_stride_head, a->lse_stride_part, a->lse_stride_part_token,
        a->out_stride_token, a->out_stride_head, a->lse_stride_token, a->lse_base2);
  } else {
    sparse_mla_merge_parts_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(a->part_out), a->part_lse, out, a->lse,
        a->s_q, a->h, a->n_parts, a->part_stride_part, a->part_stride_token, a->part_stride_head, a->lse_stride_part,
        a->lse_stride_part_token, a->out_stride_token, a->out_stride_head, a->lse_stride_token, a->lse_base2);
  }
  return check_cuda(cudaGetLastError(), "sparse_mla_merge launch");
}
