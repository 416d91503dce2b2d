// Top-k index producer: the step in front of the sparse MLA forward.  For every query token the positions of the
// `topk` largest scores among its first `length` key positions, written in ascending position order and padded
// with -1: exactly the index list the forward takes.
//
// Selection is exact and deterministic: scores are mapped to 32-bit keys whose unsigned order is the order of the
// floats (-0 below +0, NaN patterns above +inf, as an unsigned compare of the transformed bits gives), the k-th
// largest key is found by a radix select (four passes of 8 bits, a 256-bin histogram per pass in shared memory),
// and among the entries equal to that key the lowest positions are taken.  One CTA per row; the row is read from
// memory once and from L2 in the later passes, so the kernel is bound by device-memory traffic:
// 4 * s_kv bytes of scores per token (plus 4 * topk bytes of output).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flagtree_b200.h"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace topk {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

struct Params {
  const float* scores;
  const int32_t* lengths;
  int32_t* out;
  int s_q, s_kv, topk;
  long long sc_stride, out_stride;
};

__device__ __forceinline__ uint32_t to_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix of `flag` over the block in thread order; `total` = number of set flags (same in every thread)
__device__ __forceinline__ int block_exclusive(bool flag, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned b = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(b & ((1u << lane) - 1u));
  if (lane == 0) warp_sums[warp] = __popc(b);
  __syncthreads();
  int before = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int v = warp_sums[w];
    before += (w < warp) ? v : 0;
    tot += v;
  }
  __syncthreads();       // warp_sums is reused by the next call
  total = tot;
  return before + in_warp;
}

__global__ void __launch_bounds__(kThreads) topk_select_kernel(const Params p) {
  __shared__ int hist[256];
  __shared__ int warp_sums[kWarps];
  __shared__ uint32_t s_bin;
  __shared__ int s_remaining;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const float* sc = p.scores + static_cast<long long>(row) * p.sc_stride;
  int32_t* out = p.out + static_cast<long long>(row) * p.out_stride;
  int len = p.lengths != nullptr ? p.lengths[row] : p.s_kv;
  len = max(0, min(len, p.s_kv));
  const int k = min(p.topk, len);

  uint32_t thresh = 0;       // key of the k-th largest entry
  int need_eq = 0;           // how many entries equal to it are taken (the lowest positions)
  if (k < len) {
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int i = tid; i < len; i += kThreads) {
        const uint32_t key = to_key(sc[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (warp == 0) {
        // lane l owns bins 8l .. 8l + 7; walk from the largest bin down to the one that holds the `remaining`-th largest
        int mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += hist[8 * lane + j];
        int above = 0;                                   // entries in the bins of higher lanes
#pragma unroll
        for (int l = 0; l < 32; ++l) {
          const int v = __shfl_sync(0xffffffffu, mine, l);
          above += (l > lane) ? v : 0;
        }
        if (above < remaining && above + mine >= remaining) {
          int cum = above;
          for (int j = 7; j >= 0; --j) {
            const int h = hist[8 * lane + j];
            if (cum + h >= remaining) {
              s_bin = static_cast<uint32_t>(8 * lane + j);
              s_remaining = remaining - cum;
              break;
            }
            cum += h;
          }
        }
      }
      __syncthreads();
      prefix |= s_bin << shift;
      mask |= 255u << shift;
      remaining = s_remaining;
      __syncthreads();
    }
    thresh = prefix;
    need_eq = remaining;
  }

  // ordered compaction: positions in ascending order, entries above the threshold and the first need_eq equal to it
  int written = 0, eq_seen = 0;
  for (int start = 0; start < len; start += kThreads) {
    const int i = start + tid;
    bool take = false, eq = false;
    if (i < len) {
      if (k == len) {
        take = true;
      } else {
        const uint32_t key = to_key(sc[i]);
        take = key > thresh;
        eq = key == thresh;
      }
    }
    if (k < len) {
      int eq_total;
      const int eq_rank = eq_seen + block_exclusive(eq, warp_sums, eq_total);
      if (eq && eq_rank < need_eq) take = true;
      eq_seen += eq_total;
    }
    int take_total;
    const int pos = written + block_exclusive(take, warp_sums, take_total);
    if (take) out[pos] = i;
    written += take_total;
  }
  for (int j = k + tid; j < p.topk; j += kThreads) out[j] = -1;
}

}  // namespace topk
}  // namespace ftb

extern "C" FTB_API int ftb_topk_indices(const ftb_topk_args* a, void* stream) {
  using namespace ftb;
  if (a == nullptr) { set_last_error("ftb_topk_indices: args is NULL"); return FTB_ERR_INVALID; }
  if (a->s_q < 0 || a->s_kv <= 0 || a->topk <= 0) {
    set_last_error("ftb_topk_indices: bad sizes s_q=%d s_kv=%d topk=%d", a->s_q, a->s_kv, a->topk);
    return FTB_ERR_INVALID;
  }
  if (a->s_q == 0) return FTB_OK;
  if (!a->scores || !a->out) { set_last_error("ftb_topk_indices: null pointer"); return FTB_ERR_INVALID; }
  topk::Params p;
  p.scores = a->scores; p.lengths = a->lengths; p.out = a->out;
  p.s_q = a->s_q; p.s_kv = a->s_kv; p.topk = a->topk;
  p.sc_stride = a->scores_stride_token; p.out_stride = a->out_stride_token;
  topk::topk_select_kernel<<<static_cast<unsigned>(a->s_q), topk::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "ftb_topk_indices launch");
}
