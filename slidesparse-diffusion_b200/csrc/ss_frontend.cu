// Front-end: dynamic per-token INT8 quantisation + slide expansion, one pass over HBM.
//
// One CTA per token row.  A thread owns whole "chunks" of the row: CV consecutive 16-byte vectors
// (2 for 2:4, 3 for 4:6, 4 for 6:8), i.e. a whole number of groups whose slide-expanded image is a
// whole number of 16-byte vectors (16 -> 16, 24 -> 32, 32 -> 48 bytes).  The row is read once with
// 128-bit loads into registers, the absolute maximum is taken on the BF16 bit patterns (packed
// 16-bit integer max, one instruction per two elements) and reduced with warp shuffles plus one
// shared-memory hop, the row is quantised from the registers, the overlapping windows are cut
// out of the thread's own quantised bytes with funnel shifts, and written with 128-bit stores.
// No shared-memory staging of data, no re-read of x.
//
// Arithmetic follows the reference statement of the front-end exactly
// (csrc/projection_sm80.cu:8-88): absmax that ignores NaN, two IEEE divisions, an fp32 multiply
// by the reciprocal, clamp to [-128,127], round-half-even; rows m..pm-1 are zero with scale 1.
// Rows that contain Inf or NaN (detected from the same packed maximum) take an element-wise path
// that reproduces the reference's fmaxf/fminf conventions bit for bit.  No fast-math.
#include "ss_common.cuh"
#include <cuda_bf16.h>

namespace ss {
namespace {

constexpr int kMaxVec = 8;      // 16-byte vectors (8 bf16 each) a thread may hold
constexpr int kMaxThreads = 512;

__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Reference element rule, used for rows with non-finite values.
__device__ __forceinline__ uint32_t quant_exact(float v, float inv) {
  return static_cast<uint32_t>(__float2int_rn(fminf(127.f, fmaxf(-128.f, __fmul_rn(v, inv))))) & 255u;
}
__device__ __forceinline__ uint32_t quant4_exact(uint32_t a, uint32_t b, float inv) {
  return quant_exact(bf_lo(a), inv) | (quant_exact(bf_hi(a), inv) << 8) |
         (quant_exact(bf_lo(b), inv) << 16) | (quant_exact(bf_hi(b), inv) << 24);
}
// Finite rows: round to nearest even, then saturate while packing (same result as clamp-then-round).
__device__ __forceinline__ uint32_t quant4_fast(uint32_t a, uint32_t b, float inv) {
  const int i0 = __float2int_rn(__fmul_rn(bf_lo(a), inv)), i1 = __float2int_rn(__fmul_rn(bf_hi(a), inv));
  const int i2 = __float2int_rn(__fmul_rn(bf_lo(b), inv)), i3 = __float2int_rn(__fmul_rn(bf_hi(b), inv));
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(i3), "r"(i2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(i1), "r"(i0), "r"(hi));
  return out;
}

// ---- optional prologues (an extension; the reference front-end has none) -----------------------
// A prologue rewrites the row, in registers, before it is quantised, so that an element-wise
// neighbour of the projection costs no extra pass over HBM:
//   kProNormModulate  y = ((x - mean) * rstd) * (1 + scale[b]) + shift[b]   (LayerNorm without affine,
//                     then the adaLN modulation of the row's batch b = row / rows_per_batch)
//   kProGelu          y = gelu_tanh(x)
// y is rounded to BF16 and everything downstream sees exactly those BF16 values.  In
// kProNormModulate every step is a separately rounded fp32 add / multiply / divide / sqrt in a fixed
// order (no fused multiply-add), so a host restatement reproduces the result bit for bit; kProGelu
// uses the hardware tanh approximation and is reproduced within floating-point tolerance.
enum : int { kProNone = 0, kProNormModulate = 1, kProGelu = 2 };
struct Prologue {
  const uint16_t* shift;     // BF16 [batches, k], rows mod_stride elements apart
  const uint16_t* scale;     // BF16 [batches, k], rows mod_stride elements apart
  int64_t mod_stride;
  int rows_per_batch;
  float eps;
};

__device__ __forceinline__ uint32_t bf16_rn_bits(float f) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return bf16_rn_bits(lo) | (bf16_rn_bits(hi) << 16);
}
// gelu_tanh(x) = 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3), with the hardware tanh
// (tanh.approx.f32: relative error 2^-11, one special-function instruction per element; a second
// one per element would make that unit the bound of the whole kernel).  Floating point within
// tolerance: |error| <= |x| * 2.5e-4, below the BF16 rounding that follows except in the negative
// tail, where |gelu| < 4e-3 anyway.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float x2 = __fmul_rn(x, x);
  const float u = __fmul_rn(x, __fmaf_rn(x2, 0.035677408f, 0.79788456f));
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = __fmul_rn(0.5f, x);
  return __fmaf_rn(h, t, h);
}
// Block-wide sum with a fixed order: lanes by xor butterfly, then the warp totals the same way.
__device__ __forceinline__ float block_sum(float a, float* scratch, int t, int nthreads) {
#pragma unroll
  for (int d = 16; d; d >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, d));
  __syncthreads();                                   // scratch may still be read from a previous call
  if ((t & 31) == 0) scratch[t >> 5] = a;
  __syncthreads();
  float b = (t & 31) < (nthreads >> 5) ? scratch[t & 31] : 0.f;
#pragma unroll
  for (int d = 16; d; d >>= 1) b = __fadd_rn(b, __shfl_xor_sync(0xffffffffu, b, d));
  return b;
}

template <int L> struct Chunk;
template <> struct Chunk<4> { static constexpr int kVec = 2, kOutWords = 4; };
template <> struct Chunk<6> { static constexpr int kVec = 3, kOutWords = 8; };
template <> struct Chunk<8> { static constexpr int kVec = 4, kOutWords = 12; };

// Lifted words of one chunk from its quantised words (all indices are compile-time constants).
template <int L>
__device__ __forceinline__ void lift_chunk(const uint32_t* qw, uint32_t* ow) {
  constexpr int W = L / 2 - 1, kGroups = Chunk<L>::kVec * 8 / L;
#pragma unroll
  for (int g = 0; g < kGroups; ++g)
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const int o = g * L + 2 * j;                           // byte offset of the window
      ow[g * W + j] = (o & 3) ? __funnelshift_r(qw[o >> 2], qw[(o >> 2) + 1], 16) : qw[o >> 2];
    }
}

// L: group size (4, 6, 8).  VEC: rows are 16-byte aligned and k % 8 == 0.  PRO: prologue (VEC only).
template <int L, bool VEC, int PRO = kProNone>
__global__ void __launch_bounds__(kMaxThreads)
quant_lift_kernel(const uint16_t* __restrict__ x, int64_t sx, int8_t* __restrict__ q,
                  float* __restrict__ sa, int m, int k, int pk, int nvec, int nchunks, const Prologue pro) {
  constexpr int CV = Chunk<L>::kVec, OW = Chunk<L>::kOutWords, kChunks = kMaxVec / CV;
  __shared__ uint32_t warp_max[32];
  __shared__ float warp_fmax[32];
  __shared__ float s_inv;
  __shared__ uint32_t s_bits;
  // lets a GEMM launched with programmatic stream serialization run its set-up while the last
  // wave of rows is still being quantised (it waits on the device before reading q or sa)
  ptx::grid_dep_launch();

  const int row = blockIdx.x, t = threadIdx.x, T = blockDim.x;
  const bool live = row < m;
  const uint16_t* xr = x + static_cast<int64_t>(row) * sx;

  uint4 v[kChunks][CV];
  uint32_t imax = 0;                                   // packed 16-bit max of |x| bit patterns
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    if (i * T >= nchunks) break;      // no thread of the CTA owns a chunk from here on
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      const int idx = (t + i * T) * CV + c;
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
          w = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
        }
      }
      v[i][c] = w;
    }
  }
  if constexpr (PRO == kProGelu) {
#pragma unroll
    for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        uint4& w = v[i][c];
        w.x = pack_bf16(gelu_tanh(bf_lo(w.x)), gelu_tanh(bf_hi(w.x)));
        w.y = pack_bf16(gelu_tanh(bf_lo(w.y)), gelu_tanh(bf_hi(w.y)));
        w.z = pack_bf16(gelu_tanh(bf_lo(w.z)), gelu_tanh(bf_hi(w.z)));
        w.w = pack_bf16(gelu_tanh(bf_lo(w.w)), gelu_tanh(bf_hi(w.w)));
      }
  }
  if constexpr (PRO == kProNormModulate) {
    // mean and variance over the k valid elements (two passes over the registers)
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        const uint4 w = v[i][c];
        const uint32_t e[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) part = __fadd_rn(__fadd_rn(part, bf_lo(e[j])), bf_hi(e[j]));
      }
    const float kf = static_cast<float>(k);
    const float mean = __fdiv_rn(block_sum(part, warp_fmax, t, T), kf);
    part = 0.f;
#pragma unroll
    for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        if ((t + i * T) * CV + c < nvec) {
          const uint4 w = v[i][c];
          const uint32_t e[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float d0 = __fadd_rn(bf_lo(e[j]), -mean), d1 = __fadd_rn(bf_hi(e[j]), -mean);
            part = __fadd_rn(__fadd_rn(part, __fmul_rn(d0, d0)), __fmul_rn(d1, d1));
          }
        }
      }
    const float var = __fdiv_rn(block_sum(part, warp_fmax, t, T), kf);
    const float rstd = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(var, pro.eps)));
    const int64_t brow = static_cast<int64_t>(live ? row / pro.rows_per_batch : 0) * pro.mod_stride;
    const uint4* shift = reinterpret_cast<const uint4*>(pro.shift + brow);
    const uint4* scale = reinterpret_cast<const uint4*>(pro.scale + brow);
#pragma unroll
    for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        const int idx = (t + i * T) * CV + c;
        if (live && idx < nvec) {
          uint4& w = v[i][c];
          const uint4 sh = __ldg(shift + idx), sc = __ldg(scale + idx);
          uint32_t e[4] = {w.x, w.y, w.z, w.w};
          const uint32_t hs[4] = {sh.x, sh.y, sh.z, sh.w}, cs[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float y0 = __fadd_rn(__fmul_rn(__fmul_rn(__fadd_rn(bf_lo(e[j]), -mean), rstd),
                                                 __fadd_rn(1.f, bf_lo(cs[j]))), bf_lo(hs[j]));
            const float y1 = __fadd_rn(__fmul_rn(__fmul_rn(__fadd_rn(bf_hi(e[j]), -mean), rstd),
                                                 __fadd_rn(1.f, bf_hi(cs[j]))), bf_hi(hs[j]));
            e[j] = pack_bf16(y0, y1);
          }
          w = make_uint4(e[0], e[1], e[2], e[3]);
        }
      }
  }
#pragma unroll
  for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      const uint4 w = v[i][c];
      imax = __vmaxu2(imax, __vmaxu2(__vmaxu2(w.x & 0x7fff7fffu, w.y & 0x7fff7fffu),
                                     __vmaxu2(w.z & 0x7fff7fffu, w.w & 0x7fff7fffu)));
    }
#pragma unroll
  for (int d = 16; d; d >>= 1) imax = __vmaxu2(imax, __shfl_xor_sync(0xffffffffu, imax, d));
  if ((t & 31) == 0) warp_max[t >> 5] = imax;
  __syncthreads();
  if (t < 32) {
    uint32_t a = t < (T >> 5) ? warp_max[t] : 0u;
#pragma unroll
    for (int d = 16; d; d >>= 1) a = __vmaxu2(a, __shfl_xor_sync(0xffffffffu, a, d));
    if (t == 0) s_bits = max(a & 0xffffu, a >> 16);
  }
  __syncthreads();
  const uint32_t bits = s_bits;
  const bool special = bits >= 0x7f80u;                // the row holds Inf or NaN

  float amax = __uint_as_float(bits << 16);
  if (special) {
    // absolute maximum with fmaxf semantics: NaN operands are ignored, Inf wins
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < kChunks && i * T < nchunks; ++i)
#pragma unroll
      for (int c = 0; c < CV; ++c) {
        const uint4 w = v[i][c];
        a = fmaxf(a, fmaxf(fmaxf(fabsf(bf_lo(w.x)), fabsf(bf_hi(w.x))), fmaxf(fabsf(bf_lo(w.y)), fabsf(bf_hi(w.y)))));
        a = fmaxf(a, fmaxf(fmaxf(fabsf(bf_lo(w.z)), fabsf(bf_hi(w.z))), fmaxf(fabsf(bf_lo(w.w)), fabsf(bf_hi(w.w)))));
      }
#pragma unroll
    for (int d = 16; d; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    if ((t & 31) == 0) warp_fmax[t >> 5] = a;
    __syncthreads();
    a = 0.f;
    for (int i = 0; i < (T >> 5); ++i) a = fmaxf(a, warp_fmax[i]);
    amax = a;
  }
  if (t == 0) {
    const float scale = fmaxf(__fdiv_rn(fmaxf(amax, 1e-12f), 127.f), 1.f / (127.f * 512.f));
    s_inv = __fdiv_rn(1.f, scale);
    sa[row] = live ? scale : 1.f;
  }
  __syncthreads();
  const float inv = s_inv;

  uint4* qr = reinterpret_cast<uint4*>(q + static_cast<int64_t>(row) * pk);
  const int out_vecs = pk >> 4;
#pragma unroll
  for (int i = 0; i < kChunks; ++i) {
    if (i * T >= nchunks) break;      // no thread of the CTA owns a chunk from here on
    const int chunk = t + i * T;
    uint32_t qw[CV * 2 + 1], ow[OW];
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      const uint4 w = v[i][c];
      if (special) {
        qw[2 * c] = quant4_exact(w.x, w.y, inv);
        qw[2 * c + 1] = quant4_exact(w.z, w.w, inv);
      } else {
        qw[2 * c] = quant4_fast(w.x, w.y, inv);
        qw[2 * c + 1] = quant4_fast(w.z, w.w, inv);
      }
    }
    qw[CV * 2] = 0u;
    lift_chunk<L>(qw, ow);
#pragma unroll
    for (int s = 0; s < OW / 4; ++s) {
      const int ov = chunk * (OW / 4) + s;
      if (ov < out_vecs) qr[ov] = make_uint4(ow[4 * s], ow[4 * s + 1], ow[4 * s + 2], ow[4 * s + 3]);
    }
  }
}

template <int L, bool VEC, int PRO = kProNone>
int launch_one(const void* x, int64_t sx, int m, int k, int pm, int pk, int8_t* q, float* sa,
               cudaStream_t stream, const Prologue& pro = Prologue{nullptr, nullptr, 0, 1, 0.f}) {
  constexpr int CV = Chunk<L>::kVec, OW = Chunk<L>::kOutWords, kChunks = kMaxVec / CV;
  const int nvec = (k + 7) / 8;
  const int chunks_in = (nvec + CV - 1) / CV;
  const int chunks_out = ((pk >> 2) + OW - 1) / OW;     // padding words are written too
  const int chunks = chunks_in > chunks_out ? chunks_in : chunks_out;
  // a multiple of 32 threads such that threads * kChunks covers the chunks; iterations in which
  // no thread owns a chunk are skipped inside the kernel
  const int threads = ((chunks + kChunks - 1) / kChunks + 31) / 32 * 32;
  SS_REQUIRE(threads <= kMaxThreads, SS_E_LIMIT, "front-end: K=%d beyond the supported %d", k,
             kMaxThreads * kMaxVec * 8);
  quant_lift_kernel<L, VEC, PRO><<<pm, threads, 0, stream>>>(static_cast<const uint16_t*>(x), sx, q, sa, m, k, pk, nvec, chunks, pro);
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

int launch_quantize_lift_fused(const void* x, int64_t sx, int64_t m, int64_t k, int group, int prologue,
                               const void* shift, const void* scale, int64_t mod_stride,
                               int64_t rows_per_batch, float eps, int8_t* q, float* sa, cudaStream_t stream) {
  if (prologue == kProNone) return launch_quantize_lift(x, sx, m, k, group, q, sa, stream);
  SS_REQUIRE(prologue == kProNormModulate || prologue == kProGelu, SS_E_ARG, "front-end: unknown prologue %d", prologue);
  SS_REQUIRE(x && q && sa, SS_E_ARG, "front-end: null pointer");
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "front-end: group must be 4, 6 or 8 (got %d)", group);
  SS_REQUIRE(m > 0 && k > 0 && k <= 32768 && m < (1ll << 31) - 32, SS_E_ARG,
             "front-end: invalid shape m=%lld k=%lld", (long long)m, (long long)k);
  SS_REQUIRE(sx >= k, SS_E_ARG, "front-end: row stride %lld smaller than k=%lld", (long long)sx, (long long)k);
  SS_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0, SS_E_ARG, "front-end: q must be 16-byte aligned");
  SS_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (sx % 8) == 0 && (k % 8) == 0, SS_E_ARG,
             "front-end: a prologue needs 16-byte aligned rows and k %% 8 == 0");
  Prologue pro{static_cast<const uint16_t*>(shift), static_cast<const uint16_t*>(scale), mod_stride,
               static_cast<int>(rows_per_batch), eps};
  if (prologue == kProNormModulate) {
    SS_REQUIRE(shift && scale && rows_per_batch > 0 && rows_per_batch < (1ll << 31) && eps >= 0.f, SS_E_ARG,
               "front-end: norm+modulate needs shift, scale, rows_per_batch > 0 and eps >= 0");
    SS_REQUIRE(((reinterpret_cast<uintptr_t>(shift) | reinterpret_cast<uintptr_t>(scale)) & 15) == 0 &&
                   mod_stride >= k && mod_stride % 8 == 0, SS_E_ARG,
               "front-end: shift and scale rows must be 16-byte aligned (row stride >= k, multiple of 8)");
  }
  const int64_t valid = (k + group - 1) / group * (group / 2 - 1) * 4;
  const int64_t pk = ceil_to(valid, 128), pm = ceil_to(m, 32);
#define SS_DISPATCH(LL)                                                                                   \
  return prologue == kProGelu                                                                             \
             ? launch_one<LL, true, kProGelu>(x, sx, (int)m, (int)k, (int)pm, (int)pk, q, sa, stream, pro) \
             : launch_one<LL, true, kProNormModulate>(x, sx, (int)m, (int)k, (int)pm, (int)pk, q, sa, stream, pro)
  if (group == 4) { SS_DISPATCH(4); }
  if (group == 6) { SS_DISPATCH(6); }
  SS_DISPATCH(8);
#undef SS_DISPATCH
}

}  // namespace ss
