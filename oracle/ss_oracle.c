/*
 * C restatement of the sparse W8A8 projection path -- TEST INFRASTRUCTURE ONLY.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may load
 * this library; the product never does.  Plain C, exact IEEE arithmetic (built with
 * -ffp-contract=off so no multiply-add is fused behind our back; the one intended fused
 * multiply-add is the explicit fmaf of the epilogue).  Each function names the reference
 * file:line (inside the SlideSparse-Diffusion tree) whose algorithm it restates.
 *
 * Pinning status: slide and pack are pinned against the reference's own CPU code through the
 * golden vectors in tests/golden/; quantise, GEMM and epilogue are pinned against the outputs of the
 * reference's own GPU operators, recompiled for sm_100 and run on a B200 (tests/golden/ref_gpu.npz).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* cvt.rn.bf16.f32: round to nearest even, NaN -> canonical quiet NaN (0x7fff). */
static uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* sdacc/w8a8_slidesparse/packing.py:15-20 */
static int64_t lifted_valid(int64_t k, int l) { return (k + l - 1) / l * (l / 2 - 1) * 4; }

/* sdacc/w8a8_slidesparse/packing.py:23-52 (slide_weight).  Returns 0, or 1 + row of the first
 * group that breaks the (l-2):l structure. */
int64_t sso_slide_weight(const int8_t* w, int64_t n, int64_t k, int l, int8_t* out) {
  const int windows = l / 2 - 1;
  const int64_t groups = (k + l - 1) / l, valid = groups * windows * 4;
  for (int64_t r = 0; r < n; ++r)
    for (int64_t g = 0; g < groups; ++g) {
      int8_t lane[8];
      int taken[8] = {0}, nonzero = 0;
      for (int j = 0; j < l; ++j) {
        lane[j] = g * l + j < k ? w[r * k + g * l + j] : 0;
        nonzero += lane[j] != 0;
      }
      if (nonzero > l - 2) return 1 + r;
      for (int win = 0; win < windows; ++win) {
        int kept = 0;
        for (int j = 0; j < 4; ++j) {
          int p = 2 * win + j;
          int8_t v = 0;
          if (lane[p] && !taken[p] && kept < 2) { v = lane[p]; taken[p] = 1; ++kept; }
          out[r * valid + (g * windows + win) * 4 + j] = v;
        }
      }
      for (int j = 0; j < l; ++j)
        if (lane[j] && !taken[j]) return 1 + r;
    }
  return 0;
}

/* sdacc/w8a8_slidesparse/csrc/dualscale_sm80.cu:254-274 (pack_cpu before reorder_meta).
 * Returns 0, or 1 + row on a quartet with more than two nonzeros. */
int64_t sso_pack(const int8_t* w, int64_t n, int64_t kl, int64_t pk, int8_t* packed, uint32_t* raw) {
  const int64_t pn = (n + 31) / 32 * 32;
  memset(raw, 0, (size_t)(pn * (pk / 32)) * 4);
  for (int64_t r = 0; r < pn; ++r)
    for (int64_t g = 0; g < pk / 4; ++g) {
      int8_t v[4] = {0, 0, 0, 0};
      int sel[2] = {0, 0}, count = 0;
      for (int j = 0; j < 4; ++j) {
        if (r < n && g * 4 + j < kl) v[j] = w[r * kl + g * 4 + j];
        if (v[j]) {
          if (count == 2) return 1 + r;
          sel[count++] = j;
        }
      }
      for (int j = 0; count < 2 && j < 4; ++j)
        if (!v[j]) sel[count++] = j;
      if (sel[0] > sel[1]) { int t = sel[0]; sel[0] = sel[1]; sel[1] = t; }
      packed[r * (pk / 2) + 2 * g] = v[sel[0]];
      packed[r * (pk / 2) + 2 * g + 1] = v[sel[1]];
      raw[r * (pk / 32) + g / 8] |= ((uint32_t)sel[0] | ((uint32_t)sel[1] << 2)) << (4 * (g % 8));
    }
  return 0;
}

/* sdacc/w8a8_slidesparse/csrc/projection_sm80.cu:8-88 (quant_lift): x is BF16 bit patterns
 * [m, sx] (row stride sx elements), q is [pm, pk], sa is [pm]. */
void sso_quantize_lift(const uint16_t* x, int64_t sx, int64_t m, int64_t k, int l, int8_t* q, float* sa) {
  const int windows = l / 2 - 1;
  const int64_t valid = lifted_valid(k, l), pk = (valid + 127) / 128 * 128, pm = (m + 31) / 32 * 32;
  const float floor_scale = 1.f / (127.f * 512.f);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < pm; ++r) {
    int8_t* qr = q + r * pk;
    memset(qr, 0, (size_t)pk);
    if (r >= m) { sa[r] = 1.f; continue; }
    const uint16_t* xr = x + r * sx;
    float a = 0.f;
    for (int64_t c = 0; c < k; ++c) a = fmaxf(a, fabsf(bf16_to_f32(xr[c])));
    const float scale = fmaxf(fmaxf(a, 1e-12f) / 127.f, floor_scale);
    const float inv = 1.f / scale;
    sa[r] = scale;
    for (int64_t c = 0; c < valid; ++c) {
      const int64_t src = (c / (4 * windows)) * l + 2 * ((c / 4) % windows) + c % 4;
      if (src >= k) continue;
      const float v = bf16_to_f32(xr[src]) * inv;
      qr[c] = (int8_t)lrintf(fminf(127.f, fmaxf(-128.f, v)));   /* default rounding: half-even */
    }
  }
}

/* dualscale_sm80.cu:189-204: acc[m,n] = sum_c q[m,c] * lifted[n,c], exact int32. */
void sso_gemm_int32(const int8_t* q, int64_t pk, const int8_t* lifted, int64_t kl, int64_t m, int64_t n,
                    int32_t* acc) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      const int8_t* a = q + i * pk;
      const int8_t* b = lifted + j * kl;
      int32_t s = 0;
      for (int64_t c = 0; c < kl; ++c) s += (int32_t)a[c] * (int32_t)b[c];
      acc[i * n + j] = s;
    }
}

/* Same contraction from the compressed form (values + raw metadata), as the tensor core sees it. */
void sso_gemm_int32_packed(const int8_t* q, int64_t pk, const int8_t* packed, const uint32_t* raw,
                           int64_t m, int64_t n, int32_t* acc) {
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < n; ++j)
    for (int64_t i = 0; i < m; ++i) {
      const int8_t* a = q + i * pk;
      int32_t s = 0;
      for (int64_t g = 0; g < pk / 4; ++g) {
        const uint32_t nib = (raw[j * (pk / 32) + g / 8] >> (4 * (g % 8))) & 15u;
        s += (int32_t)packed[j * (pk / 2) + 2 * g] * (int32_t)a[4 * g + (nib & 3u)];
        s += (int32_t)packed[j * (pk / 2) + 2 * g + 1] * (int32_t)a[4 * g + (nib >> 2)];
      }
      acc[i * n + j] = s;
    }
}

/* dualscale_sm80.cu:72-78 (scaled<Fast=true>) and :123-135: BF16 bit patterns of
 * fma(float(acc), sa*sw, bias) (+ float(addend) as a separate fp32 add). */
void sso_epilogue(const int32_t* acc, const float* sa, const float* sw, const float* bias,
                  const uint16_t* addend, int64_t addend_stride, int64_t m, int64_t n, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      const float scale = sa[i] * sw[j];
      float y = fmaf((float)acc[i * n + j], scale, bias ? bias[j] : 0.f);
      if (addend) y = y + bf16_to_f32(addend[i * addend_stride + j]);
      out[i * n + j] = f32_to_bf16(y);
    }
}

/* Gated accumulation of the fused projection (an extension of this build, no reference
 * counterpart): out = bf16( float(residual) + float( bf16( gate[row / rows_per_batch, j] * y ) ) ),
 * y = fma(float(acc), sa*sw, bias) in fp32.  Restates the GEMM epilogue's arithmetic plus the
 * BF16 round-to-nearest add of the TMA reduction. */
void sso_epilogue_gated(const int32_t* acc, const float* sa, const float* sw, const float* bias,
                        const uint16_t* gate, int64_t gate_stride, int64_t rows_per_batch,
                        const uint16_t* residual, int64_t m, int64_t n, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      const float scale = sa[i] * sw[j];
      const float y = fmaf((float)acc[i * n + j], scale, bias ? bias[j] : 0.f);
      const float z = bf16_to_f32(f32_to_bf16(bf16_to_f32(gate[(i / rows_per_batch) * gate_stride + j]) * y));
      out[i * n + j] = f32_to_bf16(bf16_to_f32(residual[i * n + j]) + z);
    }
}

/* Fixed-order, shared-curvature pruning with joint INT8 rounding
 * (diffusion_research/reconstruction.py:55-133, compress).  w [rows,columns] is updated in place
 * to the compensated weight (dead columns must already be zero), zeros receives the selected
 * zeros, losses the proxy loss per row; upper is the shared factor [columns,columns].  Inside a
 * column block every operation is the separately rounded fp32 operation of the reference's
 * tensor expressions (:95-110; its k=1 matrix product rounds each product once); the block's
 * errors are applied to the later columns (:113-114) as acc = fma(e, u, acc) from 0 in
 * increasing k followed by one subtraction — the reference leaves the summation order of that
 * product to its BLAS, so results agree with it to rounding there.  Ties between equal scores go
 * to the lower column (torch.topk does not define them). */
static float sso_round_to_grid(float v, float s) {
  float r = rintf(v / s);
  return r < -128.f ? -128.f : (r > 127.f ? 127.f : r);
}

void sso_obs_compress(float* w, int64_t rows, int64_t columns, const float* upper, const float* scales,
                      int group, int blocksize, int joint, uint8_t* zeros, float* losses) {
  memset(zeros, 0, (size_t)(rows * columns));
  for (int64_t r = 0; r < rows; ++r) losses[r] = 0.f;
  for (int64_t start = 0; start < columns; start += blocksize) {
    const int64_t stop = start + blocksize < columns ? start + blocksize : columns;
    const int64_t width = stop - start;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      float* local = (float*)malloc(sizeof(float) * (size_t)width * 3);
      float* done = local + width;
      float* err = done + width;
      float* wr = w + r * columns;
      uint8_t* zr = zeros + r * columns;
      for (int64_t j = 0; j < width; ++j) local[j] = wr[start + j];
      for (int64_t index = 0; index < width; ++index) {
        if (index % group == 0) {
          const int64_t span = group < width - index ? group : width - index;
          const int64_t remove = 2 - (group - span) > 0 ? 2 - (group - span) : 0;
          int64_t first = -1, second = -1;
          float best = 0.f;
          for (int64_t g = 0; g < span; ++g) {
            const float v = local[index + g], d = upper[(start + index + g) * columns + start + index + g];
            const float score = (v * v) / (d * d);
            if (first < 0 || score < best) { first = g; best = score; }
          }
          if (remove > 1)
            for (int64_t g = 0; g < span; ++g) {
              if (g == first) continue;
              const float v = local[index + g], d = upper[(start + index + g) * columns + start + index + g];
              const float score = (v * v) / (d * d);
              if (second < 0 || score < best) { second = g; best = score; }
            }
          if (remove > 0) zr[start + index + first] = 1;
          if (remove > 1) zr[start + index + second] = 1;
        }
        const float current = local[index];
        float fin = joint ? sso_round_to_grid(current, scales[r]) * scales[r] : current;
        if (zr[start + index]) fin = 0.f;
        const float* frow = upper + (start + index) * columns + start;
        const float e = (current - fin) / frow[index];
        losses[r] = losses[r] + (e * e) * 0.5f;
        done[index] = fin;
        err[index] = e;
        for (int64_t j = index; j < width; ++j) local[j] = local[j] - e * frow[j];
      }
      for (int64_t j = 0; j < width; ++j) wr[start + j] = done[j];
      for (int64_t c = stop; c < columns; ++c) {
        float acc = 0.f;
        for (int64_t k = 0; k < width; ++k) acc = fmaf(err[k], upper[(start + k) * columns + c], acc);
        wr[c] = wr[c] - acc;
      }
      free(local);
    }
  }
}
