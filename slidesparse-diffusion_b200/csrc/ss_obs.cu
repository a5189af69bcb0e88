// Weight preparation on the device: the fixed-order, shared-curvature pruner with joint INT8
// rounding that produces the `qweight` / `scales` the packer consumes
// (reference: sdacc/diffusion_research/reconstruction.py:55-133, `compress`).
//
// Output rows are independent and all share one curvature factor, so a column block is processed
// by eight lanes per row: the row's slice lives in shared memory next to the block's factor tile,
// the lanes walk the columns in order (selection at each group start, rounding, error, rank-one
// update of the columns still open) and the errors of the block are then applied to all later
// columns by an fp32 GEMM with a fixed summation order.  Every floating-point operation is a
// separately rounded IEEE operation in the order the reference's tensor expressions apply them
// (the GEMM accumulates with fused multiply-adds in increasing k), which the CPU oracle repeats.
#include "ss_common.cuh"

namespace ss {
namespace {

constexpr int kObsWarps = 16;        // warps per CTA
constexpr int kLanesPerRow = 8;      // a quarter of a warp walks one row (the widest group has 8 columns)
constexpr int kRowsPerCta = kObsWarps * 32 / kLanesPerRow;

__device__ __forceinline__ float round_to_grid(float v, float s) {
  // torch.round(v / s).clamp(-128, 127): round half to even
  return fminf(127.f, fmaxf(-128.f, rintf(__fdiv_rn(v, s))));
}

// Lowest (score, column) pair of the 8 lanes that walk one row; ties go to the lower column.
__device__ __forceinline__ int argmin8(float score, int g) {
#pragma unroll
  for (int d = 4; d; d >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, score, d);
    const int other_g = __shfl_xor_sync(0xffffffffu, g, d);
    if (other < score || (other == score && other_g < g)) { score = other; g = other_g; }
  }
  return g;
}

// One column block [start, start+width).  Eight lanes walk one row: the scalar chain of a column
// (rounding, error) is repeated by those eight lanes only and the rank-one update of the columns
// still open is shared between them.  Shared memory: the upper triangle of the block's factor
// tile, row after row (row i starts at i*width - i*(i-1)/2 and holds columns i..width-1), then per
// row two float rows (open values, which become the finalised ones, and errors) and one byte row
// (selected zeros).
__global__ void __launch_bounds__(kObsWarps * 32)
obs_block_kernel(float* __restrict__ w, int rows, int64_t columns, int64_t start, int width, int rows_per_cta,
                 const float* __restrict__ upper, const float* __restrict__ scales, int group, int joint,
                 uint8_t* __restrict__ zeros, float* __restrict__ errors, float* __restrict__ losses) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* tri = reinterpret_cast<float*>(smem);
  const int tri_size = (width * (width + 1) / 2 + 3) & ~3;      // keeps the rows behind it 16-byte aligned
  const int lane = threadIdx.x & 31, sl = lane & (kLanesPerRow - 1);
  const int slot = threadIdx.x / kLanesPerRow;
  float* open = tri + tri_size + slot * 2 * width;
  float* err = open + width;
  uint8_t* chosen = reinterpret_cast<uint8_t*>(tri + tri_size + kRowsPerCta * 2 * width) + slot * width;

  for (int i = threadIdx.x; i < width * width; i += blockDim.x) {
    const int r = i / width, c = i - r * width;
    if (c >= r) tri[r * width - r * (r - 1) / 2 + c - r] = upper[(start + r) * columns + start + c];
  }
  __syncthreads();
  if ((threadIdx.x & ~31) / kLanesPerRow >= rows_per_cta) return;       // whole warp without rows

  const float inf = __int_as_float(0x7f800000);
  for (int base = blockIdx.x * rows_per_cta; base < rows; base += gridDim.x * rows_per_cta) {
    const int row = base + slot;
    const bool active = slot < rows_per_cta && row < rows;
    float* wr = w + static_cast<int64_t>(active ? row : 0) * columns + start;
    for (int j = sl; j < width; j += kLanesPerRow) { open[j] = active ? wr[j] : 0.f; chosen[j] = 0; }
    const float s = active ? scales[row] : 1.f;
    float loss = active ? losses[row] : 0.f;
    __syncwarp();
    int off = 0;                                   // where row `index` of the triangle starts
    for (int index = 0; index < width; ++index) {
      if (index % group == 0) {
        const int span = min(group, width - index);
        const int remove = max(0, 2 - (group - span));
        // the `remove` smallest scores of the group, ties to the lower column
        float score = inf;
        int g = 99;
        if (sl < span) {
          const int i = index + sl;
          const float v = open[i], d = tri[i * width - i * (i - 1) / 2];
          score = __fdiv_rn(__fmul_rn(v, v), __fmul_rn(d, d));
          g = sl;
        }
        const int first = argmin8(score, g);
        if (g == first) { score = inf; g = 99; }
        const int second = argmin8(score, g);
        if (sl == 0) {
          if (remove > 0) chosen[index + first] = 1;
          if (remove > 1) chosen[index + second] = 1;
        }
        __syncwarp();
      }
      const float current = open[index];
      float fin = joint ? __fmul_rn(round_to_grid(current, s), s) : current;
      if (chosen[index]) fin = 0.f;
      const float e = __fdiv_rn(__fsub_rn(current, fin), tri[off]);
      loss = __fadd_rn(loss, __fmul_rn(__fmul_rn(e, e), 0.5f));
      __syncwarp();
      if (sl == 0) { open[index] = fin; err[index] = e; }
      const float* frow = tri + off - index;       // frow[j] = factor[index][j] for j >= index
      if ((width & 3) == 0) {
        // four columns per lane and step: one 16-byte read and write of the open values
        float4* open4 = reinterpret_cast<float4*>(open);
        for (int q4 = ((index + 1) >> 2) + sl; q4 < (width >> 2); q4 += kLanesPerRow) {
          float4 o = open4[q4];
          const int j = q4 << 2;
          if (j > index) o.x = __fsub_rn(o.x, __fmul_rn(e, frow[j]));
          if (j + 1 > index) o.y = __fsub_rn(o.y, __fmul_rn(e, frow[j + 1]));
          if (j + 2 > index) o.z = __fsub_rn(o.z, __fmul_rn(e, frow[j + 2]));
          o.w = __fsub_rn(o.w, __fmul_rn(e, frow[j + 3]));
          open4[q4] = o;
        }
      } else {
        for (int j = index + 1 + sl; j < width; j += kLanesPerRow) open[j] = __fsub_rn(open[j], __fmul_rn(e, frow[j]));
      }
      __syncwarp();
      off += width - index;
    }
    if (active) {
      uint8_t* zr = zeros + static_cast<int64_t>(row) * columns + start;
      float* er = errors + static_cast<int64_t>(row) * width;
      for (int j = sl; j < width; j += kLanesPerRow) { wr[j] = open[j]; er[j] = err[j]; zr[j] = chosen[j]; }
      if (sl == 0) losses[row] = loss;
    }
    __syncwarp();
  }
}

// w[r, stop + j] -= sum_k errors[r, k] * upper[start + k, stop + j], the sum taken as
// acc = fma(e, u, acc) from acc = 0 in increasing k.  128 x 128 output tile, 8 x 8 per thread
// (rows ty*4+i and 64+ty*4+i, columns likewise, so shared-memory reads are conflict-free float4s),
// the next k-slab fetched into registers while the current one is multiplied.
constexpr int kTileM = 128, kTileN = 128, kTileK = 16;

__global__ void __launch_bounds__(256)
obs_trailing_kernel(float* __restrict__ w, int rows, int64_t columns, int64_t start, int width,
                    const float* __restrict__ upper, const float* __restrict__ errors) {
  __shared__ __align__(16) float a_s[kTileK][kTileM];
  __shared__ __align__(16) float b_s[kTileK][kTileN];
  const int64_t stop = start + width;
  const int cols = static_cast<int>(columns - stop);
  const int row0 = blockIdx.y * kTileM, col0 = blockIdx.x * kTileN;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  // this thread's share of a slab: 8 consecutive k of one row of A, 8 consecutive columns of one k of B
  const int a_row = t >> 1, a_k = (t & 1) * 8;
  const int b_k = t >> 4, b_col = (t & 15) * 8;
  const float* a_src = errors + static_cast<int64_t>(row0 + a_row) * width;
  const bool a_ok = row0 + a_row < rows;
  float a_reg[8], b_reg[8];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) a_reg[i] = (a_ok && k0 + a_k + i < width) ? a_src[k0 + a_k + i] : 0.f;
    const bool k_ok = k0 + b_k < width;
    const float* b_src = upper + (start + k0 + b_k) * columns + stop + col0 + b_col;
#pragma unroll
    for (int i = 0; i < 8; ++i) b_reg[i] = (k_ok && col0 + b_col + i < cols) ? b_src[i] : 0.f;
  };
  float acc[8][8] = {};
  fetch(0);
  for (int k0 = 0; k0 < width; k0 += kTileK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { a_s[a_k + i][a_row] = a_reg[i]; b_s[b_k][b_col + i] = b_reg[i]; }
    __syncthreads();
    if (k0 + kTileK < width) fetch(k0 + kTileK);
#pragma unroll
    for (int k = 0; k < kTileK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&a_s[k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&a_s[k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&b_s[k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&b_s[k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = col0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (c >= cols) continue;
      float* p = w + static_cast<int64_t>(r) * columns + stop + c;
      *p = __fsub_rn(*p, acc[i][j]);
    }
  }
}

// Final export: q = clamp(rint(w / scale)) with the selected zeros forced to 0; status bit 0 is set
// when q * scale differs from w (checked only when check_grid), bit 1 when a complete group holds
// more than group - 2 nonzeros.  One thread per (row, group).
__global__ void obs_finish_kernel(const float* __restrict__ w, const float* __restrict__ scales,
                                  const uint8_t* __restrict__ zeros, int rows, int64_t columns, int group,
                                  int check_grid, int8_t* __restrict__ q, int32_t* __restrict__ status) {
  const int64_t groups = (columns + group - 1) / group;
  const int64_t id = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (id >= rows * groups) return;
  const int64_t row = id / groups, g = id - row * groups;
  const float s = scales[row];
  int nonzero = 0, flags = 0;
  const int64_t base = row * columns;
  for (int64_t c = g * group; c < min(columns, (g + 1) * group); ++c) {
    const float v = w[base + c];
    int value = static_cast<int>(round_to_grid(v, s));
    if (zeros[base + c]) value = 0;
    q[base + c] = static_cast<int8_t>(value);
    nonzero += value != 0;
    if (check_grid && !(__fmul_rn(static_cast<float>(value), s) == v)) flags |= 1;
  }
  if ((g + 1) * group <= columns && nonzero > group - 2) flags |= 2;
  if (flags) atomicOr(status, flags);
}

}  // namespace
}  // namespace ss

using namespace ss;

static size_t obs_block_smem(int64_t width) {
  const int64_t triangle = (width * (width + 1) / 2 + 3) / 4 * 4;
  return static_cast<size_t>(triangle + kRowsPerCta * 2 * width) * sizeof(float) + kRowsPerCta * width;
}

extern "C" int ss_obs_max_blocksize(void) {
  int64_t width = 8;
  while (obs_block_smem(width + 1) <= 227 * 1024) ++width;
  return static_cast<int>(width);
}

extern "C" int ss_obs_block(float* w, int64_t rows, int64_t columns, int64_t start, int64_t width,
                            const float* upper, const float* scales, int group, int joint,
                            uint8_t* zeros, float* errors, float* losses, void* stream) {
  SS_REQUIRE(w && upper && scales && zeros && errors && losses, SS_E_ARG, "obs_block: null pointer");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "obs_block: group must be 4, 6 or 8");
  SS_REQUIRE(rows > 0 && rows < (1ll << 31) && columns > 0 && columns < (1ll << 31), SS_E_ARG, "obs_block: invalid shape");
  SS_REQUIRE(start >= 0 && width > 0 && start + width <= columns && start % group == 0, SS_E_ARG,
             "obs_block: the block [start, start+width) must lie inside the row and start on a group boundary");
  const size_t smem = obs_block_smem(width);
  SS_REQUIRE(smem <= 227 * 1024, SS_E_ARG, "obs_block: a block of %lld columns needs %zu bytes of shared memory (limit 232448)",
             static_cast<long long>(width), smem);
  SS_CUDA(cudaFuncSetAttribute(obs_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int device = 0, sms = 0;
  SS_CUDA(cudaGetDevice(&device));
  SS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // spread the rows over all SMs: a CTA takes up to kRowsPerCta rows per pass, whole warps of 4
  int64_t per_cta = ((rows + sms - 1) / sms + 3) / 4 * 4;
  if (per_cta > kRowsPerCta) per_cta = kRowsPerCta;
  const int64_t wanted = (rows + per_cta - 1) / per_cta;
  const unsigned grid = static_cast<unsigned>(wanted < sms ? wanted : sms);
  obs_block_kernel<<<grid, kObsWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      w, static_cast<int>(rows), columns, start, static_cast<int>(width), static_cast<int>(per_cta), upper, scales,
      group, joint != 0, zeros, errors, losses);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

extern "C" int ss_obs_trailing(float* w, int64_t rows, int64_t columns, int64_t start, int64_t width,
                               const float* upper, const float* errors, void* stream) {
  SS_REQUIRE(w && upper && errors, SS_E_ARG, "obs_trailing: null pointer");
  SS_REQUIRE(rows > 0 && rows < (1ll << 31) && columns > 0 && columns < (1ll << 31), SS_E_ARG, "obs_trailing: invalid shape");
  SS_REQUIRE(start >= 0 && width > 0 && start + width <= columns, SS_E_ARG, "obs_trailing: block outside the row");
  const int64_t cols = columns - start - width;
  if (cols == 0) return SS_OK;
  const dim3 grid(static_cast<unsigned>((cols + kTileN - 1) / kTileN), static_cast<unsigned>((rows + kTileM - 1) / kTileM));
  SS_REQUIRE(grid.y <= 65535, SS_E_ARG, "obs_trailing: too many rows for one launch");
  obs_trailing_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, static_cast<int>(rows), columns, start, static_cast<int>(width), upper, errors);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

extern "C" int ss_obs_finish(const float* w, const float* scales, const uint8_t* zeros, int64_t rows,
                             int64_t columns, int group, int check_grid, int8_t* qweight, int32_t* status,
                             void* stream) {
  SS_REQUIRE(w && scales && zeros && qweight && status, SS_E_ARG, "obs_finish: null pointer");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "obs_finish: group must be 4, 6 or 8");
  SS_REQUIRE(rows > 0 && rows < (1ll << 31) && columns > 0 && columns < (1ll << 31), SS_E_ARG, "obs_finish: invalid shape");
  const int64_t total = rows * ((columns + group - 1) / group);
  SS_REQUIRE((total + 255) / 256 < (1ll << 31), SS_E_ARG, "obs_finish: weight too large for one launch");
  obs_finish_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, scales, zeros, static_cast<int>(rows), columns, group, check_grid, qweight, status);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}
