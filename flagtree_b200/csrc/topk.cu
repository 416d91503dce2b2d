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


// ---------------------------------------------------------------------------------------------------------------
// Rows of at most 32768 scores: one persistent CTA of 1024 threads per SM.  The next row travels into shared
// memory by 16-byte asynchronous copies while the current one, held as 32 keys per thread in registers, is
// selected; the scores are read from device memory exactly once.  Thread t owns the 32 consecutive positions
// 32 t .. 32 t + 31 (read as eight 16-byte pieces in the order piece ^ (t & 7), which keeps the eight lanes of a
// shared-memory phase on different banks), so the ordered output needs one scan over per-thread counts and a
// walk over the few set bits of a per-thread mask.
//
// Shared-memory atomics retire about one lane per clock, so a histogram over the whole row would cost far more
// than the row takes to arrive.  A sample of 256 keys therefore brackets the k-th largest key first: the sample
// is ranked by counting, two thresholds L <= H are picked a few standard deviations of the sample quantile
// either side of rank k / len, and one sweep over the registers counts A = #{key > H} and builds a 256-bin
// histogram of key - L over the keys in [L, H].  When A < k <= A + #[L, H] (checked, so a bad sample costs time
// and never exactness) the k-th largest key lies in one bin of a few keys, which are ranked by counting;
// otherwise the sweep is repeated over the whole key range.  Bins still crowded (ties, repeated values) go
// through further 8-bit passes.  The histograms hold one counter per (bin, lane): the atomic adds of a warp fall
// into 32 different banks whatever the distribution of the scores.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kRowMax = 32768;
constexpr int kBigThreads = 1024;
constexpr int kBigWarps = kBigThreads / 32;
constexpr int kPerThread = kRowMax / kBigThreads;          // 32 keys per thread
constexpr int kSample = 256;
constexpr int kSampleMinLen = 4096;                        // shorter rows are selected without a bracket
constexpr int kListMax = 256;                              // a bin of at most this many keys is ranked by counting
constexpr size_t kBigSmem = static_cast<size_t>(kRowMax) * 4 + 256 * 32 * 4 + 256 * 4 + kSample * 4 + kBigWarps * 4 + 16 * 4 +
                            2 * kBigThreads * 4 + 2 * kListMax * 4;

enum { kCtlBin = 0, kCtlRemaining, kCtlBinCount, kCtlInside, kCtlAbove, kCtlLo, kCtlHi, kCtlListCount, kCtlThresh, kCtlNeedEq };

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ int row_len(const Params& p, int row) {
  const int len = p.lengths != nullptr ? p.lengths[row] : p.s_kv;
  return max(0, min(len, p.s_kv));
}

__device__ __forceinline__ void fetch_row(const Params& p, int row, float* buf) {
  const float* sc = p.scores + static_cast<long long>(row) * p.sc_stride;
  const int chunks = (row_len(p, row) + 3) >> 2;           // 16-byte pieces; s_kv is a multiple of 4 on this path
  for (int c = threadIdx.x; c < chunks; c += kBigThreads) cp_async16(buf + 4 * c, sc + 4 * c);
}

// moves nibble s of `bits` to nibble s ^ x (x in 0..7): register order <-> position order of a thread's keys
__device__ __forceinline__ uint32_t swap_nibbles(uint32_t bits, int x) {
  if (x & 1) bits = ((bits & 0x0f0f0f0fu) << 4) | ((bits >> 4) & 0x0f0f0f0fu);
  if (x & 2) bits = ((bits & 0x00ff00ffu) << 8) | ((bits >> 8) & 0x00ff00ffu);
  if (x & 4) bits = (bits << 16) | (bits >> 16);
  return bits;
}

__global__ void __launch_bounds__(kBigThreads, 1) topk_select_rows_kernel(const Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* buf = reinterpret_cast<float*>(smem_raw);                                   // the row in flight
  int* hist = reinterpret_cast<int*>(smem_raw + static_cast<size_t>(kRowMax) * 4);   // [256 bins][32 lanes]
  int* bin_total = hist + 256 * 32;                                                  // [256]
  uint32_t* samp = reinterpret_cast<uint32_t*>(bin_total + 256);                     // [256]
  uint32_t* warp_sum = samp + kSample;                                               // [32]
  int* ctl = reinterpret_cast<int*>(warp_sum + kBigWarps);                           // [16]
  uint32_t* gt_extra = reinterpret_cast<uint32_t*>(ctl + 16);                        // [1024] per owner thread: keys of
  uint32_t* eq_extra = gt_extra + kBigThreads;                                       // [1024] the last bin above / equal
  uint32_t* list = eq_extra + kBigThreads;                                           // [kListMax] keys of the last bin
  int* list_pos = reinterpret_cast<int*>(list + kListMax);                           // [kListMax] and their positions
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int twist = tid & 7;
  const int pos0 = tid * kPerThread;

  int row = blockIdx.x;
  if (row < p.s_q) fetch_row(p, row, buf);
  for (; row < p.s_q; row += gridDim.x) {
    const int len = row_len(p, row);
    const int k = min(p.topk, len);
    const bool sampled = k < len && len >= kSampleMinLen;
    const int n_valid = max(0, min(kPerThread, len - pos0));
    const uint32_t valid_pos = n_valid >= 32 ? 0xffffffffu : ((1u << n_valid) - 1u);   // position order
    cp_async_wait_all();
    __syncthreads();
    uint32_t key[kPerThread];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int piece = s ^ twist;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (n_valid > 0) v = *reinterpret_cast<const float4*>(buf + pos0 + 4 * piece);
      const uint32_t ok = valid_pos >> (4 * piece);          // positions past the row take the lowest key
      key[4 * s + 0] = (ok & 1u) ? to_key(v.x) : 0u;
      key[4 * s + 1] = (ok & 2u) ? to_key(v.y) : 0u;
      key[4 * s + 2] = (ok & 4u) ? to_key(v.z) : 0u;
      key[4 * s + 3] = (ok & 8u) ? to_key(v.w) : 0u;
    }
    if (sampled && tid < kSample) {
      // the sample number in the low byte makes the sample keys distinct; the bracket does not need exact keys
      const uint32_t sk = to_key(buf[static_cast<int>((static_cast<long long>(tid) * len) >> 8) + (tid & 15)]);
      samp[tid] = (sk & ~0xffu) | static_cast<uint32_t>(tid);
    }
    if (tid == 0) { ctl[kCtlLo] = 0; ctl[kCtlHi] = -1; }
    __syncthreads();
    if (row + static_cast<int>(gridDim.x) < p.s_q) fetch_row(p, row + gridDim.x, buf);   // overlaps the selection

    uint32_t above_bits = 0, tie_bits = 0;                 // register order: keys above the last bin, ties of a one-key bin
    int need_eq = 0;
    if (k < len) {
      if (sampled) {
        // rank of sample s among the 256: four threads count a quarter each
        const int s_no = tid >> 2, quarter = tid & 3;
        const uint32_t mine = samp[s_no];
        int rank = 0;
#pragma unroll
        for (int m = 0; m < kSample / 16; ++m) {           // the four threads of a sample read different banks
          const uint4 v = *reinterpret_cast<const uint4*>(samp + 16 * m + 4 * quarter);
          rank += (v.x > mine) + (v.y > mine) + (v.z > mine) + (v.w > mine);
        }
        rank += __shfl_xor_sync(0xffffffffu, rank, 1);
        rank += __shfl_xor_sync(0xffffffffu, rank, 2);
        const float frac = static_cast<float>(k) / static_cast<float>(len);
        const int centre = static_cast<int>(frac * kSample);
        const int margin = static_cast<int>(3.5f * sqrtf(kSample * frac * (1.0f - frac))) + 2;
        if (quarter == 0) {
          if (rank == centre + margin) ctl[kCtlLo] = static_cast<int>(mine & ~0xffu);   // stays 0 past the sample
          if (rank == centre - margin) ctl[kCtlHi] = static_cast<int>(mine | 0xffu);    // stays the largest key
        }
        __syncthreads();
      }
      uint32_t lo = static_cast<uint32_t>(ctl[kCtlLo]), hi = static_cast<uint32_t>(ctl[kCtlHi]);
      uint32_t cand = 0, prefix = 0, mask = 0;             // cand bit r: key[r] still in the running (register order)
      int remaining = 0, low_bits = 0, bin_count = 0;
#pragma unroll 1
      for (int attempt = 0; attempt < 2; ++attempt) {
        // first sweep: count the keys above H, histogram key - L over [L, H] in 256 bins
        const uint32_t range = hi - lo;
        low_bits = 32 - __clz(range);
        const int shift = max(low_bits - 8, 0);
        {
          int4* h4 = reinterpret_cast<int4*>(hist);
          h4[tid] = make_int4(0, 0, 0, 0);
          h4[tid + kBigThreads] = make_int4(0, 0, 0, 0);
        }
        __syncthreads();
        const uint32_t valid_reg = swap_nibbles(valid_pos, twist);
        int above = 0;
        cand = 0;
        if (valid_reg != 0) {
#pragma unroll
          for (int r = 0; r < kPerThread; ++r) {
            const uint32_t rel = key[r] - lo;
            above += key[r] > hi ? 1 : 0;
            if (rel <= range && ((valid_reg >> r) & 1u)) {
              cand |= 1u << r;
              atomicAdd(&hist[((rel >> shift) << 5) + lane], 1);
            }
          }
        }
        above = __reduce_add_sync(0xffffffffu, above);
        if (lane == 0) warp_sum[warp] = static_cast<uint32_t>(above);
        __syncthreads();
        {
          const int bin = tid >> 2, q = tid & 3;
          int t = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) t += hist[(bin << 5) + ((q * 8 + i + bin) & 31)];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          if (q == 0) bin_total[bin] = t;
        }
        __syncthreads();
        if (warp == 0) {
          const int total_above = static_cast<int>(__reduce_add_sync(0xffffffffu, warp_sum[lane]));
          int mine = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) mine += bin_total[8 * lane + j];
          int suffix = mine;                               // keys in this lane's bins and the bins of higher lanes
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_down_sync(0xffffffffu, suffix, d);
            if (lane + d < 32) suffix += v;
          }
          const int inside = __shfl_sync(0xffffffffu, suffix, 0);
          const int want = k - total_above;                // rank of the k-th largest key inside the bracket
          if (lane == 0) { ctl[kCtlAbove] = total_above; ctl[kCtlInside] = inside; }
          const int higher = suffix - mine;
          if (want > 0 && higher < want && want <= suffix) {
            int cum = higher;
            for (int j = 7; j >= 0; --j) {
              const int h = bin_total[8 * lane + j];
              if (cum + h >= want) {
                ctl[kCtlBin] = 8 * lane + j;
                ctl[kCtlRemaining] = want - cum;
                ctl[kCtlBinCount] = h;
                break;
              }
              cum += h;
            }
          }
        }
        __syncthreads();
        const int total_above = ctl[kCtlAbove];
        if (total_above < k && k <= total_above + ctl[kCtlInside]) {
          prefix = static_cast<uint32_t>(ctl[kCtlBin]) << shift;
          mask = ~((1u << shift) - 1u);                    // bits of key - L fixed so far
          remaining = ctl[kCtlRemaining];
          bin_count = ctl[kCtlBinCount];
          low_bits = shift;
          break;
        }
        lo = 0u; hi = 0xffffffffu;                         // the sample misled: select over the whole key range
      }
      // further 8-bit passes while the bin is crowded
#pragma unroll 1
      while (low_bits > 0 && bin_count > kListMax) {
        const int width = min(8, low_bits), shift = low_bits - width;
        const uint32_t digit_mask = (1u << width) - 1u;
        {
          int4* h4 = reinterpret_cast<int4*>(hist);
          h4[tid] = make_int4(0, 0, 0, 0);
          h4[tid + kBigThreads] = make_int4(0, 0, 0, 0);
        }
        __syncthreads();
        if (cand != 0) {
#pragma unroll
          for (int r = 0; r < kPerThread; ++r) {
            if ((cand >> r) & 1u) {
              const uint32_t rel = key[r] - lo;
              if ((rel & mask) == prefix) atomicAdd(&hist[(((rel >> shift) & digit_mask) << 5) + lane], 1);
              else cand &= ~(1u << r);
            }
          }
        }
        __syncthreads();
        {
          const int bin = tid >> 2, q = tid & 3;
          int t = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) t += hist[(bin << 5) + ((q * 8 + i + bin) & 31)];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          if (q == 0) bin_total[bin] = t;
        }
        __syncthreads();
        if (warp == 0) {
          int mine = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) mine += bin_total[8 * lane + j];
          int suffix = mine;
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_down_sync(0xffffffffu, suffix, d);
            if (lane + d < 32) suffix += v;
          }
          const int higher = suffix - mine;
          if (higher < remaining && remaining <= suffix) {
            int cum = higher;
            for (int j = 7; j >= 0; --j) {
              const int h = bin_total[8 * lane + j];
              if (cum + h >= remaining) {
                ctl[kCtlBin] = 8 * lane + j;
                ctl[kCtlRemaining] = remaining - cum;
                ctl[kCtlBinCount] = h;
                break;
              }
              cum += h;
            }
          }
        }
        __syncthreads();
        prefix |= static_cast<uint32_t>(ctl[kCtlBin]) << shift;
        mask |= digit_mask << shift;
        remaining = ctl[kCtlRemaining];
        bin_count = ctl[kCtlBinCount];
        low_bits = shift;
      }
      // the last bin [base, top]: keys above it are taken, its own few keys go to a list with their positions and
      // are ranked by counting: the threshold is the key v with #{keys > v} < remaining <= #{keys >= v}
      const uint32_t base = lo + prefix;
      const uint32_t span = min(low_bits == 0 ? 0u : ((1u << low_bits) - 1u), hi - base);   // keys above H were counted apart
      const uint32_t top = base + span;
      gt_extra[tid] = 0u;
      eq_extra[tid] = 0u;
      if (tid == 0) ctl[kCtlListCount] = 0;
      __syncthreads();
      const uint32_t valid_reg = swap_nibbles(valid_pos, twist);
#pragma unroll
      for (int r = 0; r < kPerThread; ++r) {
        above_bits |= key[r] > top ? (1u << r) : 0u;
        if (key[r] - base <= span && ((valid_reg >> r) & 1u)) {
          if (low_bits == 0) {
            tie_bits |= 1u << r;                           // the bin is one key wide: these are the ties
          } else {
            const int at = atomicAdd(&ctl[kCtlListCount], 1);
            list[at] = key[r];
            list_pos[at] = pos0 + 4 * ((r >> 2) ^ twist) + (r & 3);
          }
        }
      }
      need_eq = remaining;
      if (low_bits != 0) {
        __syncthreads();
        const int n = ctl[kCtlListCount];
        if (tid < n) {
          const uint32_t v = list[tid];
          int gt = 0, ge = 0;
          for (int m = 0; m < n; ++m) {
            const uint32_t o = list[m];
            gt += o > v ? 1 : 0;
            ge += o >= v ? 1 : 0;
          }
          const int at = list_pos[tid];
          if (gt < remaining) {
            if (remaining <= ge) { atomicOr(&eq_extra[at >> 5], 1u << (at & 31)); ctl[kCtlNeedEq] = remaining - gt; }
            else atomicOr(&gt_extra[at >> 5], 1u << (at & 31));
          }
        }
        __syncthreads();
        need_eq = ctl[kCtlNeedEq];
      }
    } else {
      // k == len: every position of the row is taken
      above_bits = swap_nibbles(valid_pos, twist);
      gt_extra[tid] = 0u;
      eq_extra[tid] = 0u;
      need_eq = 0;
    }

    // per thread the taken keys and the ties as bit masks in position order, one scan over the packed counts
    // (ties << 16 | taken; neither exceeds 32768), then each thread writes its few positions
    uint32_t gt_bits = swap_nibbles(above_bits, twist) | gt_extra[tid];
    uint32_t eq_bits = (swap_nibbles(tie_bits, twist) | eq_extra[tid]) & valid_pos;
    const uint32_t packed = (static_cast<uint32_t>(__popc(eq_bits)) << 16) | static_cast<uint32_t>(__popc(gt_bits));
    uint32_t incl = packed;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    const uint32_t before = __reduce_add_sync(0xffffffffu, lane < warp ? warp_sum[lane] : 0u) + incl - packed;
    const int gt_before = static_cast<int>(before & 0xffffu), eq_before = static_cast<int>(before >> 16);
    int eq_take = min(max(need_eq - eq_before, 0), __popc(eq_bits));    // the lowest positions among the ties
    uint32_t bits = gt_bits;
    while (eq_take > 0) {
      const uint32_t lowest = eq_bits & (0u - eq_bits);
      bits |= lowest;
      eq_bits ^= lowest;
      --eq_take;
    }
    int32_t* out = p.out + static_cast<long long>(row) * p.out_stride;
    int write_at = gt_before + min(eq_before, need_eq);
    while (bits != 0) {
      out[write_at++] = pos0 + __ffs(static_cast<int>(bits)) - 1;
      bits &= bits - 1u;
    }
    for (int j = k + tid; j < p.topk; j += kBigThreads) out[j] = -1;
    __syncthreads();                                       // the shared words are reused by the next row
  }
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
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool rows_path = a->s_kv <= topk::kRowMax && (a->s_kv & 3) == 0 && (a->scores_stride_token & 3) == 0 &&
                         (reinterpret_cast<uintptr_t>(a->scores) & 15) == 0;
  if (rows_path) {
    int dev = 0, sm_count = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count")) return rc;
    if (int rc = check_cuda(cudaFuncSetAttribute(topk::topk_select_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(topk::kBigSmem)), "topk shared memory")) return rc;
    const unsigned grid = static_cast<unsigned>(a->s_q < sm_count ? a->s_q : sm_count);
    topk::topk_select_rows_kernel<<<grid, topk::kBigThreads, topk::kBigSmem, st>>>(p);
  } else {
    topk::topk_select_kernel<<<static_cast<unsigned>(a->s_q), topk::kThreads, 0, st>>>(p);
  }
  return check_cuda(cudaGetLastError(), "ftb_topk_indices launch");
}
