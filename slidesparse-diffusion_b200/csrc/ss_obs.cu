// Weight preparation on the device: the fixed-order, shared-curvature pruner with joint INT8
// rounding that produces the `qweight` / `scales` the packer consumes
// (reference: sdacc/diffusion_research/reconstruction.py:55-133, `compress`).
//
// Output rows are independent and all share one curvature factor, so a column block is processed
// by one warp per row: the row's slice lives in shared memory next to the block's factor tile, the
// warp walks the columns in order (selection at each group start, rounding, error, rank-one
// update of the columns still open) and the errors of the block are then applied to all later
// columns by an fp32 GEMM with a fixed summation order.  Every floating-point operation is a
// separately rounded IEEE operation in the order the reference's tensor expressions apply them
// (the GEMM accumulates with fused multiply-adds in increasing k), which the CPU oracle repeats.
#include "ss_common.cuh"

namespace ss {
namespace {

constexpr int kObsWarps = 16;

__device__ __forceinline__ float round_to_grid(float v, float s) {
  // torch.round(v / s).clamp(-128, 127): round half to even
  return fminf(127.f, fmaxf(-128.f, rintf(__fdiv_rn(v, s))));
}

// One column block [start, start+width).  Shared memory: factor tile width x width, then per warp
// three float rows (open values, finalised values, errors) and one byte row (selected zeros).
__global__ void __launch_bounds__(kObsWarps * 32)
obs_block_kernel(float* __restrict__ w, int rows, int64_t columns, int64_t start, int width,
                 const float* __restrict__ upper, const float* __restrict__ scales, int group, int joint,
                 uint8_t* __restrict__ zeros, float* __restrict__ errors, float* __restrict__ losses) {
  extern __shared__ __align__(16) unsigned char smem[];
  float* factor = reinterpret_cast<float*>(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* open = factor + width * width + warp * 3 * width;
  float* done = open + width;
  float* err = done + width;
  uint8_t* chosen = reinterpret_cast<uint8_t*>(factor + width * width + kObsWarps * 3 * width) + warp * width;

  for (int i = threadIdx.x; i < width * width; i += blockDim.x) {
    const int r = i / width, c = i - r * width;
    factor[i] = upper[(start + r) * columns + start + c];
  }
  __syncthreads();

  for (int row = blockIdx.x * kObsWarps + warp; row < rows; row += gridDim.x * kObsWarps) {
    float* wr = w + static_cast<int64_t>(row) * columns + start;
    for (int j = lane; j < width; j += 32) { open[j] = wr[j]; chosen[j] = 0; }
    const float s = scales[row];
    float loss = losses[row];
    __syncwarp();
    for (int index = 0; index < width; ++index) {
      if (index % group == 0) {
        const int span = min(group, width - index);
        const int remove = max(0, 2 - (group - span));
        // the `remove` smallest scores of the group, ties to the lower column
        int first = -1, second = -1;
        float best = 0.f;
        for (int g = 0; g < span; ++g) {
          const float v = open[index + g], d = factor[(index + g) * width + index + g];
          const float score = __fdiv_rn(__fmul_rn(v, v), __fmul_rn(d, d));
          if (first < 0 || score < best) { first = g; best = score; }
        }
        if (remove > 1) {
          for (int g = 0; g < span; ++g) {
            if (g == first) continue;
            const float v = open[index + g], d = factor[(index + g) * width + index + g];
            const float score = __fdiv_rn(__fmul_rn(v, v), __fmul_rn(d, d));
            if (second < 0 || score < best) { second = g; best = score; }
          }
        }
        if (lane == 0) {
          if (remove > 0) chosen[index + first] = 1;
          if (remove > 1) chosen[index + second] = 1;
        }
        __syncwarp();
      }
      const float current = open[index];
      float fin = joint ? __fmul_rn(round_to_grid(current, s), s) : current;
      if (chosen[index]) fin = 0.f;
      const float e = __fdiv_rn(__fsub_rn(current, fin), factor[index * width + index]);
      loss = __fadd_rn(loss, __fmul_rn(__fmul_rn(e, e), 0.5f));
      __syncwarp();
      if (lane == 0) { done[index] = fin; err[index] = e; }
      const float* frow = factor + index * width;
      for (int j = index + lane; j < width; j += 32) open[j] = __fsub_rn(open[j], __fmul_rn(e, frow[j]));
      __syncwarp();
    }
    uint8_t* zr = zeros + static_cast<int64_t>(row) * columns + start;
    float* er = errors + static_cast<int64_t>(row) * width;
    for (int j = lane; j < width; j += 32) { wr[j] = done[j]; er[j] = err[j]; zr[j] = chosen[j]; }
    if (lane == 0) losses[row] = loss;
    __syncwarp();
  }
}

// w[r, stop + j] -= sum_k errors[r, k] * upper[start + k, stop + j], the sum taken as
// acc = fma(e, u, acc) from acc = 0 in increasing k.  64 x 64 output tile, 4 x 4 per thread.
constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

__global__ void __launch_bounds__(256)
obs_trailing_kernel(float* __restrict__ w, int rows, int64_t columns, int64_t start, int width,
                    const float* __restrict__ upper, const float* __restrict__ errors) {
  __shared__ float a_s[kTileK][kTileM + 4];
  __shared__ float b_s[kTileK][kTileN + 4];
  const int64_t stop = start + width;
  const int cols = static_cast<int>(columns - stop);
  const int row0 = blockIdx.y * kTileM, col0 = blockIdx.x * kTileN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < width; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTileM * kTileK; i += 256) {
      const int r = i / kTileK, k = i - r * kTileK;
      a_s[k][r] = (row0 + r < rows && k0 + k < width) ? errors[static_cast<int64_t>(row0 + r) * width + k0 + k] : 0.f;
    }
    for (int i = threadIdx.x; i < kTileK * kTileN; i += 256) {
      const int k = i / kTileN, c = i - k * kTileN;
      b_s[k][c] = (col0 + c < cols && k0 + k < width) ? upper[(start + k0 + k) * columns + stop + col0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTileK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = a_s[k][ty * 4 + i]; b[i] = b_s[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
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
  return static_cast<size_t>(width * width + kObsWarps * 3 * width) * sizeof(float) + kObsWarps * width;
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
  const int64_t wanted = (rows + kObsWarps - 1) / kObsWarps;
  const unsigned grid = static_cast<unsigned>(wanted < sms ? wanted : sms);
  obs_block_kernel<<<grid, kObsWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      w, static_cast<int>(rows), columns, start, static_cast<int>(width), upper, scales, group, joint != 0,
      zeros, errors, losses);
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
  obs_finish_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, scales, zeros, static_cast<int>(rows), columns, group, check_grid, qweight, status);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}
