// Sparse MLA forward for few heads (h <= 32), sm_100a: the products are taken the other way round.
//
// With 16 or 32 query heads the kernels that put the heads on the 128 rows of the MMA spend seven eighths (three
// quarters) of every tensor-core instruction on rows of zeros, and a CTA pair works on one token.  Here one CTA
// works on one token and the gathered rows are the rows of the MMA:
//
//   S^T [128 keys x NH heads]  = K_tile [128 x 576] . Q^T [576 x NH]        (36 MMAs 128 x NH x 16, A = K, B = Q)
//   O^T [512 dims x NH heads] += V_tile^T [512 x 128 keys] . P^T [128 x NH]  (4 x 8 MMAs 128 x NH x 16,
//                                                                             A = the same tile, MN-major, B = P^T)
//
// so a tile is gathered once for both products and the instructions are NH columns wide.  A score row of tensor
// memory belongs to a key: the maximum and the sum of a head are taken across the 128 threads of the four softmax
// warps (warp reductions, then four values per head through shared memory); every thread keeps the running
// maximum and sum of all NH heads.  P^T is written to the rope block of the tile, which the second product does
// not read.  Accumulators: S^T in 32 columns of tensor memory, O^T as four blocks of 32 columns (128 dims each).
//
// One tile at a time (gather with 16-byte asynchronous copies, then the products): the tile fills 144 KB of shared
// memory, there is no room for a second.  Every wait is bounded.
//
// Measured (one tile of 128 keys, h = 16, cycles of about 12 400): rows 660, issue of the 9216 copies 3400, S^T
// 2700 (36 MMAs at 75 cycles: an MMA of 16 columns takes what one of 128 takes, its time goes with the 128 rows
// of A), softmax 2600 (4900 at h = 32), O^T 2100.  2048 causal tokens with topk 2048: 0.89 ms (h = 16), 1.14 ms
// (h = 32) against 0.80 ms for the persistent CTA pairs with the heads zero-padded to 128 rows, which therefore
// stay the default; this kernel is selected with algo_id 2.
#include <cstring>

#include "sm100.cuh"
#include "../../include/flagtree_b200.h"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace mla_few {

constexpr int kDqk = 576;
constexpr int kNChunk = 9;
constexpr int kNT = 128;                       // gathered rows per tile = rows of the MMAs
constexpr int kKvBlock = kNT * 128;            // 16384: [128 rows x 128 B], one 64-column block of the tile
constexpr int kKvBytes = kNChunk * kKvBlock;   // 147456
constexpr int kThreads = 256;
constexpr uint32_t kColS = 0;                  // tensor memory: S^T, then four O^T blocks, 32 columns each
constexpr uint32_t kColO = 32;
constexpr uint32_t kTmemCols = 256;

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
  unsigned long long bar_s;     // S^T of the tile is complete
  unsigned long long bar_o;     // O^T has taken the tile in
  uint32_t tmem_base;
  int abort_flag;
  int n_scan;
  int bad_index;
  uint32_t valid_mask[4];       // 128 validity bits of the tile
  int rows[kNT];                // row of the cache for each row of the tile (0 when masked)
  int wmax[4][32];              // per softmax warp and head: maximum of the warp's 32 keys (order-preserving integer)
  float wsum[4][32];            // per softmax warp and head: sum of the warp's 32 probabilities
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// floats <-> integers whose signed order is the order of the floats
__device__ __forceinline__ int to_ordered(float x) {
  const int i = __float_as_int(x);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float from_ordered(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

template <int NH>
__global__ void __launch_bounds__(kThreads, 1) sparse_mla_few_heads_kernel(const Params p) {
  constexpr int kQBlock = NH * 128;             // [NH heads x 128 B]
  constexpr int kQBytes = kNChunk * kQBlock;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw_addr);
  const uint32_t kv_s = base;
  const uint32_t q_s = base + kKvBytes;
  const uint32_t p_s = kv_s + 8 * kKvBlock;     // P^T [2 blocks of 64 keys][NH heads x 128 B] over the rope block
  Misc* misc = reinterpret_cast<Misc*>(sm + kKvBytes + kQBytes);
  const uint32_t bar_s = smem_u32(&misc->bar_s);
  const uint32_t bar_o = smem_u32(&misc->bar_o);
  volatile int* abort_flag = &misc->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int token = blockIdx.x;

  if (tid == 0) {
    misc->abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    misc->n_scan = 0;
    misc->bad_index = 0;
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (misc->abort_flag) return;   // an earlier launch on this status word failed: do nothing
  if (warp == 0) {
    tmem_alloc(smem_u32(&misc->tmem_base), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  // number of leading top-k slots that must be visited (last non-negative entry + 1)
  {
    int local = 0;
    const int32_t* idx_row = p.indices + static_cast<long long>(token) * p.idx_st;
    for (int j = tid; j < p.topk; j += kThreads)
      if (idx_row[j] >= 0) local = j + 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = max(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0 && local > 0) atomicMax(&misc->n_scan, local);
  }
  // Q of the token -> shared memory, K-major blocks [NH rows x 128 B] (rows at and above h are zero)
  {
    const __nv_bfloat16* q_tok = p.q + static_cast<long long>(token) * p.q_st;
    for (int c = tid; c < NH * (kDqk / 8); c += kThreads) {
      const int r = c / (kDqk / 8);
      const int ch = c - r * (kDqk / 8);
      const uint32_t dst = q_s + (ch >> 3) * kQBlock + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
      if (r < p.h) cp_async16(dst, q_tok + static_cast<long long>(r) * p.q_sh + ch * 8);
      else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
    }
    cp_async_commit();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc->tmem_base;
  const int n_tiles = (misc->n_scan + kNT - 1) / kNT;

  constexpr uint32_t kIdescQK = umma_idesc(kFmtBF16, 128, NH, 0, 0);   // A = K rows (K-major), B = Q (K-major)
  constexpr uint32_t kIdescPV = umma_idesc(kFmtBF16, 128, NH, 1, 0);   // A = V^T (MN-major), B = P^T (K-major)

  // running maximum (log2 domain) and sum of every head, kept by each of the 128 softmax threads
  float m_run[NH], l_run[NH];
#pragma unroll
  for (int hh = 0; hh < NH; ++hh) { m_run[hh] = -INFINITY; l_run[hh] = 0.0f; }

  for (int tile = 0; tile < n_tiles; ++tile) {
    const uint32_t parity = tile & 1;
    // ---- rows of this tile
    if (tid < kNT) {
      const int j = tile * kNT + tid;
      int logical = -1;
      if (j < p.topk) logical = p.indices[static_cast<long long>(token) * p.idx_st + j];
      const bool ok = logical >= 0 && logical < p.s_kv;
      if (logical < -1 || logical >= p.s_kv) misc->bad_index = 1;      // reported, never read
      misc->rows[tid] = ok ? logical : 0;
      const uint32_t m = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) misc->valid_mask[warp] = m;
    }
    __syncthreads();
    // ---- gather: 128 rows x 72 pieces of 16 bytes into nine swizzled blocks
    for (int c = tid; c < kNT * (kDqk / 8); c += kThreads) {
      const int r = c / (kDqk / 8);
      const int ch = c - r * (kDqk / 8);
      const uint32_t dst = kv_s + (ch >> 3) * kKvBlock + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
      cp_async16(dst, p.kv + static_cast<long long>(misc->rows[r]) * p.kv_sr + ch * 8);
    }
    cp_async_commit();
    cp_async_wait_all();
    fence_proxy_async_smem();
    __syncthreads();

    // ---- S^T = K . Q^T
    if (tid == 0) {
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < kNChunk; ++cc) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t ad = smem_desc_sw128(kv_s + cc * kKvBlock + k * 32, 16, 1024);
          const uint64_t bd = smem_desc_sw128(q_s + cc * kQBlock + k * 32, 16, 1024);
          umma_f16_ss(tmem + kColS, ad, bd, kIdescQK, (cc | k) != 0 ? 1u : 0u);
        }
      }
      umma_commit(bar_s);
    }

    // ---- softmax: thread = key (row of S^T), all heads
    if (warp < 4) {
      mbar_wait(bar_s, parity, abort_flag);
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, kColS), sr);
      tmem_wait_ld();
      const bool valid = (misc->valid_mask[warp] >> lane) & 1u;
      // The reductions of the heads are independent of one another: all of them are issued before any result is
      // used (a loop that took a head through its reduction before the next one cost 400 cycles a head).
      {
        int wm[NH];
#pragma unroll
        for (int hh = 0; hh < NH; ++hh)
          wm[hh] = __reduce_max_sync(0xffffffffu, valid ? to_ordered(__uint_as_float(sr[hh])) : static_cast<int>(0x80000000u));
        if (lane == 0) {
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) misc->wmax[warp][hh] = wm[hh];
        }
      }
      named_bar_sync(1, 128);
      float alpha[NH], ps[NH];
      bool moved = false;
      // this key's place in P^T: block of 64 keys, 16-byte piece within the head's row, element within the piece
      const uint32_t p_key = p_s + (tid >> 6) * kQBlock + (tid & 7) * 2;
      const int piece = (tid & 63) >> 3;
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) {
        const int t = max(max(misc->wmax[0][hh], misc->wmax[1][hh]), max(misc->wmax[2][hh], misc->wmax[3][hh]));
        const float mx = t == static_cast<int>(0x80000000u) ? -INFINITY : from_ordered(t);
        const float m_new = fmaxf(m_run[hh], mx * p.scale_log2);
        const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
        alpha[hh] = (m_run[hh] == -INFINITY) ? 0.0f : fast_exp2(m_run[hh] - m_use);
        moved = moved || alpha[hh] != 1.0f;
        m_run[hh] = m_new;
        const float pv = valid ? fast_exp2(fmaf(__uint_as_float(sr[hh]), p.scale_log2, -m_use)) : 0.0f;
        ps[hh] = pv;
        const uint32_t bits = pack_bf16x2(pv, 0.0f) & 0xffffu;
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(p_key + hh * 128 + ((piece ^ (hh & 7)) << 4)), "h"(static_cast<unsigned short>(bits)) : "memory");
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) ps[hh] += __shfl_xor_sync(0xffffffffu, ps[hh], o);
      }
      if (lane == 0) {
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) misc->wsum[warp][hh] = ps[hh];
      }
      named_bar_sync(1, 128);
#pragma unroll
      for (int hh = 0; hh < NH; ++hh)
        l_run[hh] = l_run[hh] * alpha[hh] + ((misc->wsum[0][hh] + misc->wsum[1][hh]) + (misc->wsum[2][hh] + misc->wsum[3][hh]));
      // O^T [dim][head] *= alpha[head] when a maximum moved (every thread holds the same factors: uniform)
      if (tile > 0 && moved) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_addr(tmem, warp * 32, kColO + 32 * c), o);
          tmem_wait_ld();
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) o[hh] = __float_as_uint(__uint_as_float(o[hh]) * alpha[hh]);
          tmem_st32(tmem_addr(tmem, warp * 32, kColO + 32 * c), o);
        }
        tmem_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before();
    }
    __syncthreads();

    // ---- O^T += V^T . P^T  (four blocks of 128 dims, eight steps of 16 keys)
    if (tid == 0) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t ad = smem_desc_sw128(kv_s + (2 * c) * kKvBlock + k * 2048, kKvBlock, 1024);
          const uint64_t bd = smem_desc_sw128(p_s + (k >> 2) * kQBlock + (k & 3) * 32, 16, 1024);
          umma_f16_ss(tmem + kColO + 32 * c, ad, bd, kIdescPV, (tile != 0 || k != 0) ? 1u : 0u);
        }
      }
      umma_commit(bar_o);
    }
    // the tile's shared memory and O^T are reused by the next iteration: wait for the MMAs
    mbar_wait(bar_o, parity, abort_flag);
    tc_fence_after();
  }
  cp_async_wait_all();   // Q's copies, when the token has no tile at all

  // ---- epilogue: out[head][dim] = O^T[dim][head] / l[head]; thread = dim within a block of 128
  if (warp < 4) {
    float inv_l[NH];
#pragma unroll
    for (int hh = 0; hh < NH; ++hh) inv_l[hh] = l_run[hh] > 0.0f ? 1.0f / l_run[hh] : 0.0f;
    __nv_bfloat16* o_tok = p.out + static_cast<long long>(token) * p.out_st;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      if (n_tiles > 0) {
        tmem_ld32(tmem_addr(tmem, warp * 32, kColO + 32 * c), o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int hh = 0; hh < 32; ++hh) o[hh] = 0u;
      }
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) {
        if (hh < p.h) {
          const uint32_t bits = pack_bf16x2(__uint_as_float(o[hh]) * inv_l[hh], 0.0f) & 0xffffu;
          reinterpret_cast<unsigned short*>(o_tok + static_cast<long long>(hh) * p.out_sh)[128 * c + tid] = static_cast<unsigned short>(bits);
        }
      }
    }
#pragma unroll
    for (int hh = 0; hh < NH; ++hh) {
      if (hh == tid && hh < p.h) {
        const float l2 = l_run[hh] > 0.0f ? m_run[hh] + log2f(l_run[hh]) : -INFINITY;
        p.lse[static_cast<long long>(token) * p.lse_st + hh] = (p.lse_base2 || l2 == -INFINITY) ? l2 : l2 * 0.6931471805599453f;
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

template <int NH>
static int launch_nh(const Params& p, cudaStream_t st) {
  constexpr int smem = kKvBytes + kNChunk * NH * 128 + static_cast<int>(sizeof(Misc)) + 1024;
  auto kern = sparse_mla_few_heads_kernel<NH>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(sparse_mla few heads)");
  kern<<<static_cast<unsigned>(p.s_q), kThreads, smem, st>>>(p);
  return check_cuda(cudaGetLastError(), "sparse_mla few heads launch");
}

}  // namespace mla_few

// bf16 form, plain indices, h <= 32 (argument checks are the caller's: ftb_sparse_mla_fwd)
int launch_sparse_mla_few(const ftb_sparse_mla_args* a, cudaStream_t st) {
  mla_few::Params p;
  memset(&p, 0, sizeof(p));
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
  if (a->h <= 16) return mla_few::launch_nh<16>(p, st);
  return mla_few::launch_nh<32>(p, st);
}

}  // namespace ftb
