// Per-head norms of an attention layer's projections, with the rotation and the cache write.
//
// gg_qkv_norm_rope_write, for row t = [nh heads of q | nkv heads of k | nv heads of v]:
//   q_h <- rot(q_h / rms(q_h) * wq)                        in place (the attention reads it there)
//   k_g <- rot(k_g / rms(k_g) * wk)                        to kcache [pages, nkv, page, d] at slot[t]
//   v_g <- v_g / rms(v_g)            (v_unit)              to vcache [pages, nv, page, dv]
//   v_g <- (1 - lam) v_g + lam v_first[t, g]  (mix == 2),  or  v_first[t, g] <- v_g  (mix == 1)
// rms(x) = sqrt(mean(x^2) + eps) over the head; wq, wk are one weight vector [d] for all heads, or
// null for no norm.  rot turns the first `rot` values of a head by position * inv_freq[i], pairs
// (2i, 2i+1) if interleaved, else (i, i + rot/2); cosines and sines times `mag`.  v_first is a
// float32 buffer [T, nv*dv] that lives for one step: the first layer of a model that blends values
// across layers fills it, the later ones read it.  Statistics, weights, angles and the blend are
// float32 (the angle is reduced in float64); results are rounded once, to the activation type.
#include "common.cuh"

#define HN_WARPS 4

template <typename TA>
__global__ void __launch_bounds__(HN_WARPS * 32)
qkv_norm_rope_write_kernel(TA* __restrict__ qkv, long long row_stride, const int* __restrict__ positions,
                           const int* __restrict__ slot_mapping, const double* __restrict__ inv_freq, float mag,
                           const float* __restrict__ wq, const float* __restrict__ wk, float eps, int v_unit,
                           int mix, float lam, float* __restrict__ v_first, TA* __restrict__ kcache,
                           TA* __restrict__ vcache, int nh, int nkv, int d, int nv, int dv, int rot, int page_size,
                           int interleaved, int write_cache) {
  extern __shared__ float cs[];        // cos[rot/2], sin[rot/2]
  pdl_trigger();
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (inv_freq) {
    const double pos = (double)positions[t];
    const double two_pi = 6.283185307179586476925286766559;
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
      const double ang = pos * inv_freq[p];
      const float r = (float)(ang - two_pi * rint(ang * (1.0 / two_pi)));
      float s, c;
      sincosf(r, &s, &c);
      cs[p] = c * mag;
      cs[half + p] = s * mag;
    }
  }
  const int slot = (write_cache && slot_mapping) ? slot_mapping[t] : -1;
  __syncthreads();
  pdl_wait();
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  TA* row = qkv + (size_t)t * row_stride;
  const int nrot = inv_freq ? half : 0;
  for (int h = blockIdx.y * HN_WARPS + warp; h < nh + nkv + nv; h += gridDim.y * HN_WARPS) {
    if (h < nh + nkv) {
      TA* x = row + (size_t)h * d;
      const float* w = h < nh ? wq : wk;
      float rinv = 1.f;
      if (w) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) { const float v = to_f32(x[c]); ss += v * v; }
        rinv = rsqrtf(warp_sum(ss) / (float)d + eps);
      }
      TA* kc = (h >= nh && slot >= 0) ? kcache + (((size_t)page * nkv + (h - nh)) * page_size + off) * d : nullptr;
      for (int p = lane; p < nrot; p += 32) {
        const int i0 = interleaved ? 2 * p : p;
        const int i1 = interleaved ? 2 * p + 1 : p + half;
        const float u = to_f32(x[i0]) * rinv * (w ? w[i0] : 1.f), v = to_f32(x[i1]) * rinv * (w ? w[i1] : 1.f);
        const float c = cs[p], s = cs[half + p];
        const TA ru = from_f32<TA>(u * c - v * s);
        const TA rv = from_f32<TA>(v * c + u * s);
        x[i0] = ru;
        x[i1] = rv;
        if (kc) { kc[i0] = ru; kc[i1] = rv; }
      }
      for (int c = 2 * nrot + lane; c < d; c += 32) {
        const TA y = w ? from_f32<TA>(to_f32(x[c]) * rinv * w[c]) : x[c];
        if (w) x[c] = y;
        if (kc) kc[c] = y;
      }
    } else {
      const int hv = h - nh - nkv;
      const TA* x = row + (size_t)(nh + nkv) * d + (size_t)hv * dv;
      float rinv = 1.f;
      if (v_unit) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) { const float v = to_f32(x[c]); ss += v * v; }
        rinv = rsqrtf(warp_sum(ss) / (float)dv + eps);
      }
      TA* vcp = slot >= 0 ? vcache + (((size_t)page * nv + hv) * page_size + off) * dv : nullptr;
      float* vf = v_first ? v_first + ((size_t)t * nv + hv) * dv : nullptr;
      for (int c = lane; c < dv; c += 32) {
        float v = to_f32(x[c]) * rinv;
        if (mix == 2) v = (1.f - lam) * v + lam * vf[c];
        else if (mix == 1) vf[c] = v;
        if (vcp) vcp[c] = from_f32<TA>(v);
      }
    }
  }
}

extern "C" int gg_qkv_norm_rope_write(void* qkv, long long row_stride, int act_dtype, const int* positions,
                                      const int* slot_mapping, const double* inv_freq, float mag, const float* wq,
                                      const float* wk, float eps, int v_unit, int mix, float lam, float* v_first,
                                      void* kcache, void* vcache, int T, int nh, int nkv, int d, int nv, int dv,
                                      int rot, int page_size, int interleaved, int write_cache, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && d > 0 && nv > 0 && dv > 0 && page_size > 0,
             "qkv_norm_rope_write: bad sizes T=%d nh=%d nkv=%d d=%d nv=%d dv=%d page=%d", T, nh, nkv, d, nv, dv, page_size);
  GG_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "qkv_norm_rope_write: rotary width %d must be even and <= head size %d", rot, d);
  GG_REQUIRE(row_stride >= (long long)(nh + nkv) * d + (long long)nv * dv, "qkv_norm_rope_write: rows of %lld values are too short", row_stride);
  GG_REQUIRE(!write_cache || (kcache && vcache && slot_mapping), "qkv_norm_rope_write: cache write without cache or slots");
  GG_REQUIRE(mix >= 0 && mix <= 2 && (mix == 0 || v_first), "qkv_norm_rope_write: blending values needs the buffer of the first layer's");
  GG_REQUIRE(eps >= 0.f, "qkv_norm_rope_write: eps %g", (double)eps);
  if (T == 0) return GG_OK;
  if (rot == 0) inv_freq = nullptr;
  const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
  const int heads = nh + nkv + nv;
  int gy = (heads + HN_WARPS - 1) / HN_WARPS;
  if (gy > 1024) gy = 1024;
  const dim3 grid(T, gy);
  if (act_dtype == GG_F32)
    gg_launch(qkv_norm_rope_write_kernel<float>, grid, dim3(HN_WARPS * 32), smem, stream, (float*)qkv, row_stride, positions,
              slot_mapping, inv_freq, mag, wq, wk, eps, v_unit, mix, lam, v_first, (float*)kcache, (float*)vcache, nh, nkv, d,
              nv, dv, rot, page_size, interleaved, write_cache);
  else if (act_dtype == GG_BF16)
    gg_launch(qkv_norm_rope_write_kernel<__nv_bfloat16>, grid, dim3(HN_WARPS * 32), smem, stream, (__nv_bfloat16*)qkv, row_stride,
              positions, slot_mapping, inv_freq, mag, wq, wk, eps, v_unit, mix, lam, v_first, (__nv_bfloat16*)kcache,
              (__nv_bfloat16*)vcache, nh, nkv, d, nv, dv, rot, page_size, interleaved, write_cache);
  else
    return gg_fail(GG_ERR_INVALID, "qkv_norm_rope_write: unknown dtype %d", act_dtype);
  return gg_check_launch("qkv_norm_rope_write");
}
