// Offline weight packer: (l-2):l slide expansion, 2:4 compression, metadata, weight grid.
//
// Host versions mirror the reference's CPU preparation path (packing.py:23-52 and
// csrc/dualscale_sm80.cu:254-274) so PackedLinear.prepare works without a GPU; the device
// versions do the same work in one pass for weights that already live in HBM.
#include "ss_common.cuh"
#include <cstring>
#include <vector>

namespace ss {
namespace {

// Greedy window allocation for one group of l lanes (lanes >= remaining read as zero):
// window w looks at lanes [2w, 2w+4) and keeps the first two nonzero lanes that no earlier
// window took.  Writes W*4 lifted values.  Returns false if a nonzero lane stays unallocated.
__host__ __device__ inline bool slide_group(const int8_t* base, int remaining, int l, int8_t* out) {
  const int windows = l / 2 - 1;
  unsigned taken = 0;
  int nonzero = 0;
  int8_t lanes[8];
  for (int j = 0; j < l; ++j) {
    lanes[j] = j < remaining ? base[j] : int8_t(0);
    nonzero += lanes[j] != 0;
  }
  if (nonzero > l - 2) return false;
  for (int w = 0; w < windows; ++w) {
    int kept = 0;
    for (int j = 0; j < 4; ++j) {
      const int lane = 2 * w + j;
      int8_t value = 0;
      if (lanes[lane] != 0 && !(taken & (1u << lane)) && kept < 2) {
        value = lanes[lane];
        taken |= 1u << lane;
        ++kept;
      }
      out[w * 4 + j] = value;
    }
  }
  for (int j = 0; j < l; ++j)
    if (lanes[j] != 0 && !(taken & (1u << j))) return false;
  return true;
}

// One quartet -> two kept values and the 4-bit index pair (nonzero lanes first, then the
// lowest-index zero lanes, sorted).  Returns false if more than two lanes are nonzero.
__host__ __device__ inline bool compress_quartet(const int8_t v[4], int8_t kept[2], uint32_t* nibble) {
  int sel[2] = {0, 0}, count = 0;
  for (int j = 0; j < 4; ++j)
    if (v[j]) {
      if (count == 2) return false;
      sel[count++] = j;
    }
  for (int j = 0; count < 2 && j < 4; ++j)
    if (!v[j]) sel[count++] = j;
  if (sel[0] > sel[1]) { int s = sel[0]; sel[0] = sel[1]; sel[1] = s; }
  kept[0] = v[sel[0]];
  kept[1] = v[sel[1]];
  *nibble = static_cast<uint32_t>(sel[0]) | (static_cast<uint32_t>(sel[1]) << 2);
  return true;
}

__host__ __device__ inline int64_t b200_word_index(int64_t row, int64_t col, int64_t pk) {
  return ((row >> 5) * (pk >> 7) + (col >> 2)) * 128 + (row & 31) * 4 + (col & 3);
}

// ---- device kernels ----------------------------------------------------------------------

// One thread per (row, metadata word) = 8 quartets = 32 lifted columns.
template <int L>
__global__ void pack_kernel(const int8_t* __restrict__ qweight, int n, int k, int pn, int pk,
                            int8_t* __restrict__ packed, uint32_t* __restrict__ meta,
                            int32_t* __restrict__ status) {
  constexpr int W = L / 2 - 1;
  const int words = pk >> 5;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<int64_t>(pn) * words) return;
  const int row = static_cast<int>(gid / words), col = static_cast<int>(gid % words);
  const int groups = (k + L - 1) / L;
  uint32_t word = 0;
  uint4 values = make_uint4(0u, 0u, 0u, 0u);
  uint32_t* vw = reinterpret_cast<uint32_t*>(&values);
  int cached_group = -1;
  int8_t lifted[W * 4];
  bool bad = false;
#pragma unroll
  for (int qi = 0; qi < 8; ++qi) {
    const int window = col * 8 + qi;          // global window (= quartet) index in the row
    const int g = window / W, w = window % W;
    int8_t quartet[4] = {0, 0, 0, 0};
    if (row < n && g < groups) {
      if (g != cached_group) {
        const int8_t* base = qweight + static_cast<int64_t>(row) * k + static_cast<int64_t>(g) * L;
        const int remaining = k - g * L;
        bad |= !slide_group(base, remaining, L, lifted);
        cached_group = g;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) quartet[j] = lifted[w * 4 + j];
    }
    int8_t kept[2];
    uint32_t nibble;
    bad |= !compress_quartet(quartet, kept, &nibble);
    word |= nibble << (4 * qi);
    const uint32_t pair = static_cast<uint32_t>(static_cast<uint8_t>(kept[0])) |
                          (static_cast<uint32_t>(static_cast<uint8_t>(kept[1])) << 8);
    vw[qi >> 1] |= pair << (16 * (qi & 1));
  }
  reinterpret_cast<uint4*>(packed + static_cast<int64_t>(row) * (pk >> 1))[col] = values;
  meta[b200_word_index(row, col, pk)] = word;
  if (bad) atomicOr(status, 1);
}

// One CTA per row: scale = 2*absmax/255 (1 for an all-zero row), q = clamp(rint(w/scale)).
__global__ void weight_grid_kernel(const float* __restrict__ w, int k, int8_t* __restrict__ q,
                                   float* __restrict__ scales) {
  __shared__ float warp_max[32];
  __shared__ float s_scale;
  const int row = blockIdx.x, t = threadIdx.x;
  const float* wr = w + static_cast<int64_t>(row) * k;
  float amax = 0.f;
  for (int c = t; c < k; c += blockDim.x) amax = fmaxf(amax, fabsf(wr[c]));
  for (int d = 16; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  if ((t & 31) == 0) warp_max[t >> 5] = amax;
  __syncthreads();
  if (t == 0) {
    float a = 0.f;
    for (int i = 0; i < (blockDim.x + 31) / 32; ++i) a = fmaxf(a, warp_max[i]);
    const float s = __fdiv_rn(__fmul_rn(a, 2.f), 255.f);
    s_scale = s == 0.f ? 1.f : s;
    scales[row] = s_scale;
  }
  __syncthreads();
  const float s = s_scale;
  int8_t* qr = q + static_cast<int64_t>(row) * k;
  for (int c = t; c < k; c += blockDim.x)
    qr[c] = static_cast<int8_t>(__float2int_rn(fminf(127.f, fmaxf(-128.f, __fdiv_rn(wr[c], s)))));
}

}  // namespace
}  // namespace ss

using namespace ss;

extern "C" int ss_lifted_k(int64_t k, int group, int64_t* valid, int64_t* pk) {
  SS_REQUIRE(k > 0 && mode_ok(group), SS_E_ARG, "lifted_k: positive K and group 4/6/8 required");
  const int64_t v = (k + group - 1) / group * (group / 2 - 1) * 4;
  if (valid) *valid = v;
  if (pk) *pk = ceil_to(v, 128);
  return SS_OK;
}

extern "C" int ss_slide_weight_cpu(const int8_t* qweight, int64_t n, int64_t k, int group,
                                   int8_t* lifted) {
  SS_REQUIRE(qweight && lifted, SS_E_ARG, "slide_weight: null pointer");
  SS_REQUIRE(n > 0 && k > 0, SS_E_ARG, "slide_weight: empty weights are unsupported");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "slide_weight: format must be 2:4, 4:6, or 6:8");
  const int l = group, windows = l / 2 - 1;
  const int64_t groups = (k + l - 1) / l, valid = groups * windows * 4;
  for (int64_t row = 0; row < n; ++row) {
    const int8_t* src = qweight + row * k;
    int8_t* dst = lifted + row * valid;
    for (int64_t g = 0; g < groups; ++g) {
      const int64_t remaining = k - g * l;
      const int8_t* base = src + g * l;
      const bool ok = slide_group(base, static_cast<int>(remaining < l ? remaining : l), l,
                                  dst + g * windows * 4);
      SS_REQUIRE(ok, SS_E_FORMAT, "weight violates the frozen (L-2):L structure (row %lld, group %lld)",
                 (long long)row, (long long)g);
    }
  }
  return SS_OK;
}

extern "C" int ss_pack_cpu(const int8_t* lifted, int64_t n, int64_t kl, int64_t pk, int8_t* packed,
                           int32_t* meta_raw, int32_t* meta_b200) {
  SS_REQUIRE(lifted && packed, SS_E_ARG, "pack: null pointer");
  SS_REQUIRE(n > 0 && kl > 0 && pk >= kl && pk % 128 == 0, SS_E_ARG, "pack: invalid 128-K padding");
  const int64_t pn = ceil_to(n, 32), words = pk / 32;
  for (int64_t row = 0; row < pn; ++row) {
    for (int64_t c = 0; c < words; ++c) {
      uint32_t word = 0;
      for (int qi = 0; qi < 8; ++qi) {
        const int64_t g = c * 8 + qi;
        int8_t quartet[4] = {0, 0, 0, 0};
        if (row < n)
          for (int j = 0; j < 4; ++j)
            if (g * 4 + j < kl) quartet[j] = lifted[row * kl + g * 4 + j];
        int8_t kept[2];
        uint32_t nibble;
        SS_REQUIRE(compress_quartet(quartet, kept, &nibble), SS_E_FORMAT,
                   "more than 2 nonzeros in a frozen 2:4 group (row %lld, quartet %lld)",
                   (long long)row, (long long)g);
        packed[row * (pk / 2) + 2 * g] = kept[0];
        packed[row * (pk / 2) + 2 * g + 1] = kept[1];
        word |= nibble << (4 * qi);
      }
      if (meta_raw) meta_raw[row * words + c] = static_cast<int32_t>(word);
      if (meta_b200) meta_b200[b200_word_index(row, c, pk)] = static_cast<int32_t>(word);
    }
  }
  return SS_OK;
}

extern "C" int ss_meta_convert(const int32_t* src, int32_t* dst, int64_t pn, int64_t pk, int to_b200) {
  SS_REQUIRE(src && dst && src != dst, SS_E_ARG, "meta_convert: distinct non-null buffers required");
  SS_REQUIRE(pn > 0 && pn % 32 == 0 && pk > 0 && pk % 128 == 0, SS_E_ARG,
             "meta_convert: pn must be a multiple of 32 and pk of 128");
  const int64_t words = pk / 32;
  for (int64_t row = 0; row < pn; ++row)
    for (int64_t c = 0; c < words; ++c) {
      const int64_t raw = row * words + c, hw = b200_word_index(row, c, pk);
      if (to_b200) dst[hw] = src[raw]; else dst[raw] = src[hw];
    }
  return SS_OK;
}

extern "C" int ss_weight_grid_device(const float* w, int64_t n, int64_t k, int8_t* qweight,
                                     float* scales, void* stream) {
  SS_REQUIRE(w && qweight && scales, SS_E_ARG, "weight_grid: null pointer");
  SS_REQUIRE(n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31), SS_E_ARG, "weight_grid: invalid shape");
  weight_grid_kernel<<<static_cast<unsigned>(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, static_cast<int>(k), qweight, scales);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

extern "C" int ss_pack_device(const int8_t* qweight, int64_t n, int64_t k, int group, int8_t* packed,
                              int32_t* meta_b200, int32_t* status, void* stream) {
  SS_REQUIRE(qweight && packed && meta_b200 && status, SS_E_ARG, "pack_device: null pointer");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "pack_device: group must be 4, 6 or 8");
  SS_REQUIRE(n > 0 && k > 0 && n < (1ll << 30) && k <= (1 << 20), SS_E_ARG, "pack_device: invalid shape");
  SS_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 15) == 0, SS_E_ARG, "pack_device: packed must be 16-byte aligned");
  int64_t valid, pk;
  ss_lifted_k(k, group, &valid, &pk);
  const int64_t pn = ceil_to(n, 32), total = pn * (pk / 32);
  const int threads = 128;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  auto s = static_cast<cudaStream_t>(stream);
  uint32_t* meta = reinterpret_cast<uint32_t*>(meta_b200);
  if (group == 4) pack_kernel<4><<<blocks, threads, 0, s>>>(qweight, (int)n, (int)k, (int)pn, (int)pk, packed, meta, status);
  else if (group == 6) pack_kernel<6><<<blocks, threads, 0, s>>>(qweight, (int)n, (int)k, (int)pn, (int)pk, packed, meta, status);
  else pack_kernel<8><<<blocks, threads, 0, s>>>(qweight, (int)n, (int)k, (int)pn, (int)pk, packed, meta, status);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}
