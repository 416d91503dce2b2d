// Write path of the paged FP8 latent cache: new latent rows (bf16, 576 values) are quantised to e4m3 with
// one fp32 scale per page and scattered into their slots.  This is the producer of the format that the paged
// sparse-MLA forward reads (value = e4m3 * kv_scale[page]).
//
// Rule for the page scale.  kv_scale[page] == 0 marks a page that holds nothing yet.  A call raises the scale
// of every page it touches to  max(old scale, max|new rows of the page| / 448)  (never below 1e-12 / 448), and
// when that raises the scale of a page that already held rows (old scale > 0), the 64 x 576 bytes of the page
// are requantised in place,  e4m3(decode(byte) * old / new),  before the new rows are written with the new
// scale.  Filling a page in one call therefore gives exactly amax / 448 over the page and one rounding per
// value; filling it in several calls gives the same scale and at most one extra rounding per raise.
//
// Three small kernels per call, all bound by device-memory traffic (1152 B read + 576 B written per row):
//   1. one warp per new row: row maximum -> atomicMax on the page's candidate scale (a caller workspace of
//      4 bytes per page, cleared first);
//   2. one CTA per page: untouched pages leave at once, touched pages settle their scale and requantise;
//   3. one warp per new row: quantise with the settled scale and write the 576 bytes.
// The division x / scale is the IEEE one, as in the CPU restatement, so bytes and scales agree bit for bit.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flagtree_b200.h"

namespace ftb {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

namespace kvw {

constexpr int kD = 576;
constexpr float kE4m3Max = 448.0f;

struct Params {
  const __nv_bfloat16* rows;
  const int32_t* slots;
  uint8_t* cache;
  float* scale;
  unsigned int* cand;       // workspace: candidate scale per page as float bits (non-negative floats order as integers)
  int n_rows, num_pages, page_size;
  long long row_stride;     // elements between new rows
  int* status;
};

__device__ __forceinline__ float decode_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float scale) {
  const float v[4] = {a, b, c, d};
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q = __fdiv_rn(v[i], scale);
    q = fminf(fmaxf(q, -kE4m3Max), kE4m3Max);
    out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  }
  return out;
}

// lane l of the warp holds bf16 values 8l .. 8l+7 and 256+8l .. (two 16-byte loads) and, for l < 8, 512+8l ..
__device__ __forceinline__ void load_row(const __nv_bfloat16* src, int lane, uint4 (&v)[3]) {
  v[0] = *reinterpret_cast<const uint4*>(src + 8 * lane);
  v[1] = *reinterpret_cast<const uint4*>(src + 256 + 8 * lane);
  v[2] = lane < 8 ? *reinterpret_cast<const uint4*>(src + 512 + 8 * lane) : make_uint4(0, 0, 0, 0);
}
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(256) row_amax_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= p.n_rows) return;
  const int slot = p.slots[r];
  if (slot < 0) return;                                   // -1: the row is not stored
  const int page = slot / p.page_size;
  if (page >= p.num_pages) {
    if (lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, FTB_ERR_BAD_INDEX);
    return;
  }
  uint4 v[3];
  load_row(p.rows + static_cast<long long>(r) * p.row_stride, lane, v);
  float mx = 0.0f;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float f[8];
    unpack8(v[k], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) {
    const float cand = __fdiv_rn(fmaxf(mx, 1e-12f), kE4m3Max);
    atomicMax(p.cand + page, __float_as_uint(cand));
  }
}

__global__ void __launch_bounds__(256) page_settle_kernel(const Params p) {
  const int page = blockIdx.x;
  const unsigned int cb = p.cand[page];
  if (cb == 0u) return;                                   // no new row for this page
  const float cand = __uint_as_float(cb);
  const float old = p.scale[page];
  if (!(cand > old)) return;                              // the page's scale already covers the new rows
  __syncthreads();                                        // every thread has read the old scale
  if (old > 0.0f) {
    // the page held rows under a smaller scale: bring its bytes to the new one
    uint32_t* words = reinterpret_cast<uint32_t*>(p.cache + static_cast<long long>(page) * p.page_size * kD);
    const int n_words = p.page_size * kD / 4;
    for (int i = threadIdx.x; i < n_words; i += blockDim.x) {
      const uint32_t w = words[i];
      uint32_t o = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        float q = __fdiv_rn(decode_e4m3(static_cast<uint8_t>(w >> (8 * b))) * old, cand);
        q = fminf(fmaxf(q, -kE4m3Max), kE4m3Max);
        o |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * b);
      }
      words[i] = o;
    }
  }
  if (threadIdx.x == 0) p.scale[page] = cand;
}

__global__ void __launch_bounds__(256) row_store_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= p.n_rows) return;
  const int slot = p.slots[r];
  if (slot < 0) return;
  const int page = slot / p.page_size;
  if (page >= p.num_pages) return;                        // reported by the first kernel
  const float scale = p.scale[page];
  uint4 v[3];
  load_row(p.rows + static_cast<long long>(r) * p.row_stride, lane, v);
  uint8_t* dst = p.cache + static_cast<long long>(slot) * kD;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    if (k == 2 && lane >= 8) break;
    float f[8];
    unpack8(v[k], f);
    uint2 o;
    o.x = quant4(f[0], f[1], f[2], f[3], scale);
    o.y = quant4(f[4], f[5], f[6], f[7], scale);
    *reinterpret_cast<uint2*>(dst + k * 256 + 8 * lane) = o;
  }
}

}  // namespace kvw
}  // namespace ftb

extern "C" FTB_API int64_t ftb_kv_cache_write_workspace_bytes(int32_t num_pages) {
  return num_pages > 0 ? static_cast<int64_t>(num_pages) * 4 : 0;
}

extern "C" FTB_API int ftb_kv_cache_write_fp8(const ftb_kv_cache_write_args* a, void* stream) {
  using namespace ftb;
  if (a == nullptr) { set_last_error("ftb_kv_cache_write_fp8: args is NULL"); return FTB_ERR_INVALID; }
  if (a->n_rows < 0 || a->num_pages <= 0 || a->page_size <= 0) {
    set_last_error("ftb_kv_cache_write_fp8: bad sizes n_rows=%d num_pages=%d page_size=%d", a->n_rows, a->num_pages, a->page_size);
    return FTB_ERR_INVALID;
  }
  if (a->n_rows == 0) return FTB_OK;
  if (!a->rows || !a->slot_mapping || !a->kv_cache || !a->kv_scale || !a->workspace) {
    set_last_error("ftb_kv_cache_write_fp8: null pointer");
    return FTB_ERR_INVALID;
  }
  if ((reinterpret_cast<uintptr_t>(a->rows) & 15) || (a->row_stride % 8) || (reinterpret_cast<uintptr_t>(a->kv_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 3)) {
    set_last_error("ftb_kv_cache_write_fp8: rows and kv_cache must be 16-byte aligned, row_stride a multiple of 8 elements");
    return FTB_ERR_INVALID;
  }
  if (a->workspace_bytes < ftb_kv_cache_write_workspace_bytes(a->num_pages)) {
    set_last_error("ftb_kv_cache_write_fp8: workspace of %lld bytes, ftb_kv_cache_write_workspace_bytes() asks for %lld",
                   static_cast<long long>(a->workspace_bytes), static_cast<long long>(ftb_kv_cache_write_workspace_bytes(a->num_pages)));
    return FTB_ERR_INVALID;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  kvw::Params p;
  p.rows = reinterpret_cast<const __nv_bfloat16*>(a->rows);
  p.slots = a->slot_mapping;
  p.cache = reinterpret_cast<uint8_t*>(a->kv_cache);
  p.scale = a->kv_scale;
  p.cand = reinterpret_cast<unsigned int*>(a->workspace);
  p.n_rows = a->n_rows; p.num_pages = a->num_pages; p.page_size = a->page_size;
  p.row_stride = a->row_stride;
  p.status = a->status;
  cudaError_t e = cudaMemsetAsync(p.cand, 0, static_cast<size_t>(a->num_pages) * 4, st);
  if (e != cudaSuccess) return check_cuda(e, "ftb_kv_cache_write_fp8: cudaMemsetAsync");
  const unsigned row_blocks = static_cast<unsigned>((static_cast<long long>(a->n_rows) * 32 + 255) / 256);
  kvw::row_amax_kernel<<<row_blocks, 256, 0, st>>>(p);
  kvw::page_settle_kernel<<<static_cast<unsigned>(a->num_pages), 256, 0, st>>>(p);
  kvw::row_store_kernel<<<row_blocks, 256, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "ftb_kv_cache_write_fp8 launch");
}
