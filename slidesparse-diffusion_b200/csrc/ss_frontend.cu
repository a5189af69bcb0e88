// Front-end: dynamic per-token INT8 quantisation + slide expansion, one pass over HBM.
//
// One CTA per token row.  The row is read once with 128-bit loads and kept in registers
// (up to kMaxVec 16-byte vectors per thread), the absolute maximum is reduced with warp shuffles
// (plus one shared-memory hop between warps), and the row is quantised from the registers.
// For 2:4 the quantised bytes go straight to global memory; for 4:6 / 6:8 they pass through a
// shared-memory copy of the row from which every thread assembles 16-byte vectors of the
// overlapping-window layout, so the lifted row is written with full 16-byte stores.
//
// Arithmetic follows the reference statement of the front-end exactly
// (csrc/projection_sm80.cu:8-88): fmaxf absmax that ignores NaN, two IEEE divisions, an fp32
// multiply by the reciprocal, clamp to [-128,127], round-half-even; rows m..pm-1 are zero with
// scale 1.  No fast-math.
#include "ss_common.cuh"

namespace ss {
namespace {

constexpr int kMaxVec = 8;      // 16-byte vectors (8 bf16 each) a thread may hold
constexpr int kMaxThreads = 512;

__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t quant1(float v, float inv) {
  return static_cast<uint32_t>(__float2int_rn(fminf(127.f, fmaxf(-128.f, __fmul_rn(v, inv))))) &
         255u;
}
__device__ __forceinline__ uint32_t quant_pair_lo(uint32_t a, uint32_t b, float inv) {
  // four consecutive bf16 (two packed words) -> four int8 in one word
  return quant1(bf_lo(a), inv) | (quant1(bf_hi(a), inv) << 8) | (quant1(bf_lo(b), inv) << 16) |
         (quant1(bf_hi(b), inv) << 24);
}

// L: group size (4, 6, 8).  VEC: rows are 16-byte aligned and k % 8 == 0.
template <int L, bool VEC>
__global__ void __launch_bounds__(kMaxThreads)
quant_lift_kernel(const uint16_t* __restrict__ x, int64_t sx, int8_t* __restrict__ q,
                  float* __restrict__ sa, int m, int k, int pk, int nvec) {
  extern __shared__ __align__(16) uint8_t qs[];   // L != 4: quantised row, un-lifted
  __shared__ float warp_max[32];
  __shared__ float s_inv;

  const int row = blockIdx.x, t = threadIdx.x, T = blockDim.x;
  const bool live = row < m;
  const uint16_t* xr = x + static_cast<int64_t>(row) * sx;

  uint4 v[kMaxVec];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int idx = t + i * T;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (live && idx < nvec) {
      if constexpr (VEC) {
        w = __ldg(reinterpret_cast<const uint4*>(xr) + idx);
      } else {
        uint32_t e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int col = idx * 8 + j;
          e[j] = col < k ? static_cast<uint32_t>(__ldg(xr + col)) : 0u;
        }
        w = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16),
                       e[6] | (e[7] << 16));
      }
    }
    v[i] = w;
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(w.x)), fabsf(bf_hi(w.x))),
                             fmaxf(fabsf(bf_lo(w.y)), fabsf(bf_hi(w.y)))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(w.z)), fabsf(bf_hi(w.z))),
                             fmaxf(fabsf(bf_lo(w.w)), fabsf(bf_hi(w.w)))));
  }
#pragma unroll
  for (int d = 16; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  if ((t & 31) == 0) warp_max[t >> 5] = amax;
  __syncthreads();
  if (t < 32) {
    float a = t < (T >> 5) ? warp_max[t] : 0.f;
#pragma unroll
    for (int d = 16; d; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    if (t == 0) {
      const float scale = fmaxf(__fdiv_rn(fmaxf(a, 1e-12f), 127.f), 1.f / (127.f * 512.f));
      s_inv = __fdiv_rn(1.f, scale);
      sa[row] = live ? scale : 1.f;
    }
  }
  __syncthreads();
  const float inv = s_inv;

  int8_t* qr = q + static_cast<int64_t>(row) * pk;
  if constexpr (L == 4) {
    // lifted row == quantised row, zero-padded to pk
    const int nout = pk >> 3;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int idx = t + i * T;
      if (idx < nout) {
        uint2 o = make_uint2(quant_pair_lo(v[i].x, v[i].y, inv), quant_pair_lo(v[i].z, v[i].w, inv));
        if (!live) o = make_uint2(0u, 0u);
        reinterpret_cast<uint2*>(qr)[idx] = o;
      }
    }
  } else {
    constexpr int W = L / 2 - 1;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int idx = t + i * T;
      if (idx < nvec) {
        uint2 o = make_uint2(quant_pair_lo(v[i].x, v[i].y, inv), quant_pair_lo(v[i].z, v[i].w, inv));
        if (!live) o = make_uint2(0u, 0u);
        reinterpret_cast<uint2*>(qs)[idx] = o;
      }
    }
    if (t < 4) reinterpret_cast<uint32_t*>(qs + nvec * 8)[t] = 0u;   // tail-group lanes >= k
    __syncthreads();
    const int valid_words = (k + L - 1) / L * W;
    const int nout = pk >> 4;
    for (int ov = t; ov < nout; ov += T) {
      uint32_t word[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int w = ov * 4 + j;
        uint32_t value = 0u;
        if (w < valid_words) {
          const int src = (w / W) * L + 2 * (w % W);      // even byte offset
          const uint16_t* p = reinterpret_cast<const uint16_t*>(qs + src);
          value = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 16);
        }
        word[j] = value;
      }
      reinterpret_cast<uint4*>(qr)[ov] = make_uint4(word[0], word[1], word[2], word[3]);
    }
  }
}

template <int L, bool VEC>
int launch_one(const void* x, int64_t sx, int m, int k, int pm, int pk, int8_t* q, float* sa,
               cudaStream_t stream) {
  const int nvec = (k + 7) / 8;
  const int need = L == 4 ? (pk >> 3) : nvec;       // vectors the register loop must cover
  int threads = 32;
  while (threads * kMaxVec < need) threads <<= 1;
  SS_REQUIRE(threads <= kMaxThreads, SS_E_LIMIT, "front-end: K=%d beyond the supported %d", k,
             kMaxThreads * kMaxVec * 8);
  const size_t smem = L == 4 ? 0 : static_cast<size_t>(nvec) * 8 + 16;
  auto kernel = quant_lift_kernel<L, VEC>;
  if (smem > 48 * 1024) {
    static thread_local int configured_device = -1;
    int dev = 0;
    SS_CUDA(cudaGetDevice(&dev));
    if (configured_device != dev) {
      SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
      configured_device = dev;
    }
  }
  kernel<<<pm, threads, smem, stream>>>(static_cast<const uint16_t*>(x), sx, q, sa, m, k, pk, nvec);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

}  // namespace

int launch_quantize_lift(const void* x, int64_t sx, int64_t m, int64_t k, int group, int8_t* q,
                         float* sa, cudaStream_t stream) {
  SS_REQUIRE(x && q && sa, SS_E_ARG, "front-end: null pointer");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "front-end: group must be 4, 6 or 8 (got %d)", group);
  SS_REQUIRE(m > 0 && k > 0 && k <= 32768 && m < (1ll << 31) - 32, SS_E_ARG,
             "front-end: invalid shape m=%lld k=%lld", (long long)m, (long long)k);
  SS_REQUIRE(sx >= k, SS_E_ARG, "front-end: row stride %lld smaller than k=%lld", (long long)sx,
             (long long)k);
  const int64_t valid = (k + group - 1) / group * (group / 2 - 1) * 4;
  const int64_t pk = ceil_to(valid, 128), pm = ceil_to(m, 32);
  SS_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0, SS_E_ARG, "front-end: q must be 16-byte aligned");
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (sx % 8) == 0 && (k % 8) == 0;
#define SS_DISPATCH(LL)                                                                       \
  return vec ? launch_one<LL, true>(x, sx, (int)m, (int)k, (int)pm, (int)pk, q, sa, stream)   \
             : launch_one<LL, false>(x, sx, (int)m, (int)k, (int)pm, (int)pk, q, sa, stream)
  if (group == 4) { SS_DISPATCH(4); }
  if (group == 6) { SS_DISPATCH(6); }
  SS_DISPATCH(8);
#undef SS_DISPATCH
}

}  // namespace ss
