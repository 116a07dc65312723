// The latent of a latent-attention mixer: one row per token from which every head's keys and
// values are expanded, and the only thing its cache holds.
//
// gg_latent_norm_write: c[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w, x[t] = columns
// [col0, col0 + R) of row t of the projection output; c goes, rounded to the cache's type, to
// the paged cache [pages, 1, page_size, Rp] at slot_mapping[t] (Rp >= R: the columns past R are
// written as zeros, so that a kernel which reads rows of Rp values sees R values and padding).
// Statistics and the product with the weight are float32.
//
// gg_act: element-wise activations of a plain (ungated) feed-forward.
#include "common.cuh"

template <typename TA>
__global__ void latent_norm_write_kernel(const TA* __restrict__ src, long long src_stride, int col0, int R,
                                         int Rp, const float* __restrict__ w, float eps,
                                         const int* __restrict__ slots, TA* __restrict__ cache) {
  __shared__ float red[33];
  pdl_trigger();
  const int t = blockIdx.x;
  const int slot = slots[t];                       // the step's packed list: copied in before the step began
  pdl_wait();
  if (slot < 0) return;                            // padding of a captured step: nothing to keep
  const TA* x = src + (size_t)t * src_stride + col0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    const float v = to_f32(x[c]);
    ss += v * v;
  }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)R + eps);
  TA* o = cache + (size_t)slot * Rp;
  for (int c = threadIdx.x; c < Rp; c += blockDim.x)
    o[c] = c < R ? from_f32<TA>(to_f32(x[c]) * rinv * w[c]) : from_f32<TA>(0.f);
}

extern "C" int gg_latent_norm_write(const void* src, long long src_stride, int col0, int R, int Rp,
                                    const float* w, float eps, const int* slots, void* cache,
                                    int act_dtype, int T, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && R > 0 && Rp >= R && col0 >= 0 && src_stride >= col0 + R,
             "latent_norm_write: bad sizes T=%d R=%d Rp=%d col0=%d stride=%lld", T, R, Rp, col0, src_stride);
  GG_REQUIRE(src && w && slots && cache, "latent_norm_write: a pointer is null");
  if (T == 0) return GG_OK;
  const int threads = R >= 512 ? 256 : 128;
  if (act_dtype == GG_F32)
    gg_launch(latent_norm_write_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)src, src_stride, col0,
              R, Rp, w, eps, slots, (float*)cache);
  else if (act_dtype == GG_BF16)
    gg_launch(latent_norm_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)src,
              src_stride, col0, R, Rp, w, eps, slots, (__nv_bfloat16*)cache);
  else
    return gg_fail(GG_ERR_INVALID, "latent_norm_write: unknown dtype %d", act_dtype);
  return gg_check_launch("latent_norm_write");
}

// The rotated part of a latent attention whose keys have, beside what is expanded from the latent, `rot`
// values that carry the position and are shared by all heads.  For token t: the key part (columns
// [k_col0, k_col0 + rot) of the projection row) is rotated and written to columns [dst_col, dst_col + rot)
// of the cache row at slot[t] (rows of `row` values; the latent occupies the columns before), and every
// head's query part (columns [h * q_head + q_off, + rot) of the row) is rotated and written to columns
// [h * row + dst_col, + rot) of qout[t].  Pairs (2i, 2i+1) if interleaved, else (i, i + rot/2); cosines
// and sines times mag; the angle is reduced in float64.
template <typename TA>
__global__ void latent_rope_kernel(const TA* __restrict__ src, long long src_stride, int k_col0, int q_head, int q_off,
                                   int H, int rot, const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float mag, int interleaved, const int* __restrict__ slots, TA* __restrict__ cache,
                                   TA* __restrict__ qout, long long q_stride, int row, int dst_col, int write_cache) {
  extern __shared__ float cs[];        // cos[rot/2], sin[rot/2]
  pdl_trigger();
  const int t = blockIdx.x, half = rot >> 1;
  {
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
  const int slot = (write_cache && slots) ? slots[t] : -1;
  __syncthreads();
  pdl_wait();
  const TA* x = src + (size_t)t * src_stride;
  // unit 0: the key part; unit 1 + h: head h's query part
  for (int e = threadIdx.x; e < (H + 1) * half; e += blockDim.x) {
    const int unit = e / half, p = e - unit * half;
    const int i0 = interleaved ? 2 * p : p, i1 = interleaved ? 2 * p + 1 : p + half;
    const TA* in = unit == 0 ? x + k_col0 : x + (size_t)(unit - 1) * q_head + q_off;
    TA* out = unit == 0 ? (slot >= 0 ? cache + (size_t)slot * row + dst_col : nullptr)
                        : qout + (size_t)t * q_stride + (size_t)(unit - 1) * row + dst_col;
    if (!out) continue;
    const float u = to_f32(in[i0]), v = to_f32(in[i1]);
    const float c = cs[p], s = cs[half + p];
    out[i0] = from_f32<TA>(u * c - v * s);
    out[i1] = from_f32<TA>(v * c + u * s);
  }
}

extern "C" int gg_latent_rope(const void* src, long long src_stride, int k_col0, int q_head, int q_off, int H, int rot,
                              const int* positions, const double* inv_freq, float mag, int interleaved, const int* slots,
                              void* cache, void* qout, long long q_stride, int row, int dst_col, int write_cache,
                              int act_dtype, int T, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && rot > 0 && rot % 2 == 0 && dst_col >= 0 && dst_col + rot <= row,
             "latent_rope: bad sizes T=%d H=%d rot=%d row=%d col=%d", T, H, rot, row, dst_col);
  GG_REQUIRE(src && positions && inv_freq && qout && q_stride >= (long long)H * row, "latent_rope: a pointer is null or the query rows are too short");
  GG_REQUIRE(!write_cache || (cache && slots), "latent_rope: cache write without cache or slots");
  if (T == 0) return GG_OK;
  const size_t smem = (size_t)rot * sizeof(float);
  GG_REQUIRE(smem <= 48 * 1024, "latent_rope: rotary width %d too large", rot);
  if (act_dtype == GG_F32)
    gg_launch(latent_rope_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)src, src_stride, k_col0, q_head, q_off, H,
              rot, positions, inv_freq, mag, interleaved, slots, (float*)cache, (float*)qout, q_stride, row, dst_col, write_cache);
  else if (act_dtype == GG_BF16)
    gg_launch(latent_rope_kernel<__nv_bfloat16>, dim3(T), dim3(128), smem, stream, (const __nv_bfloat16*)src, src_stride, k_col0,
              q_head, q_off, H, rot, positions, inv_freq, mag, interleaved, slots, (__nv_bfloat16*)cache, (__nv_bfloat16*)qout,
              q_stride, row, dst_col, write_cache);
  else
    return gg_fail(GG_ERR_INVALID, "latent_rope: unknown dtype %d", act_dtype);
  return gg_check_launch("latent_rope");
}

// a[t, h * n .. h * n + n) *= sigmoid(gates[t, col0 + h]): the output gate of an attention head, for
// steps whose per-head products ran in the vendor library.
template <typename TA>
__global__ void head_gate_kernel(TA* __restrict__ a, const TA* __restrict__ gates, long long ldg, int col0, int H, int n) {
  pdl_trigger();
  pdl_wait();
  __shared__ float gs[1024];                     // the token's gates, sigmoid applied (launcher: H <= 1024)
  const size_t t = blockIdx.x;
  const int w = H * n;
  for (int h = threadIdx.x; h < H; h += blockDim.x) gs[h] = 1.f / (1.f + expf(-to_f32(gates[t * ldg + col0 + h])));
  __syncthreads();
  if (n % 2 == 0 && sizeof(TA) == 2) {           // bfloat16 pairs: both values of a pair belong to one head
    __nv_bfloat162* row = reinterpret_cast<__nv_bfloat162*>(a + t * w);
    for (int c = threadIdx.x; c < w / 2; c += blockDim.x) {
      const float g = gs[(2 * c) / n];
      const float2 v = __bfloat1622float2(row[c]);
      row[c] = __floats2bfloat162_rn(v.x * g, v.y * g);
    }
    return;
  }
  for (int c = threadIdx.x; c < w; c += blockDim.x) a[t * w + c] = from_f32<TA>(to_f32(a[t * w + c]) * gs[c / n]);
}

extern "C" int gg_head_gate(void* a, const void* gates, long long ldg, int col0, int T, int H, int n, int act_dtype,
                            cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && H <= 1024 && n > 0 && a && gates, "head_gate: bad arguments (at most 1024 heads)");
  if (T == 0) return GG_OK;
  if (act_dtype == GG_F32)
    gg_launch(head_gate_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)a, (const float*)gates, ldg, col0, H, n);
  else if (act_dtype == GG_BF16)
    gg_launch(head_gate_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)a, (const __nv_bfloat16*)gates, ldg, col0, H, n);
  else
    return gg_fail(GG_ERR_INVALID, "head_gate: unknown dtype %d", act_dtype);
  return gg_check_launch("head_gate");
}

// kind 0: relu(z)^2;  1: gelu, tanh form: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)));  2: silu
enum { GG_ACT_RELU2 = 0, GG_ACT_GELU_TANH = 1, GG_ACT_SILU = 2 };

__device__ __forceinline__ float act_apply(float z, int kind) {
  if (kind == GG_ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
  if (kind == GG_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

template <typename TA>
__global__ void act_kernel(const TA* __restrict__ in, TA* __restrict__ out, size_t n, int kind) {
  pdl_trigger();
  pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x)
    out[e] = from_f32<TA>(act_apply(to_f32(in[e]), kind));
}

// 16 bytes a thread (n a multiple of the chunk, both pointers 16-byte aligned)
template <typename TA>
__global__ void act_vec_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t chunks, int kind) {
  constexpr int VPT = 16 / (int)sizeof(TA);
  pdl_trigger();
  pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < chunks; e += (size_t)gridDim.x * blockDim.x) {
    uint4 r = in[e];
    TA* v = reinterpret_cast<TA*>(&r);
#pragma unroll
    for (int j = 0; j < VPT; ++j) v[j] = from_f32<TA>(act_apply(to_f32(v[j]), kind));
    out[e] = r;
  }
}

extern "C" int gg_act(const void* in, void* out, int act_dtype, long long n, int kind, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && in && out, "act: bad arguments");
  GG_REQUIRE(kind >= 0 && kind <= 2, "act: unknown activation %d", kind);
  if (n == 0) return GG_OK;
  const int vpt = act_dtype == GG_F32 ? 4 : 8;
  if ((act_dtype == GG_F32 || act_dtype == GG_BF16) && n % vpt == 0 && ((size_t)in % 16) == 0 && ((size_t)out % 16) == 0) {
    const long long chunks = n / vpt;
    long long vb = (chunks + 255) / 256;
    if (vb > 148 * 32) vb = 148 * 32;
    if (act_dtype == GG_F32)
      gg_launch(act_vec_kernel<float>, dim3((int)vb), dim3(256), 0, stream, (const uint4*)in, (uint4*)out, (size_t)chunks, kind);
    else
      gg_launch(act_vec_kernel<__nv_bfloat16>, dim3((int)vb), dim3(256), 0, stream, (const uint4*)in, (uint4*)out, (size_t)chunks, kind);
    return gg_check_launch("act");
  }
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (act_dtype == GG_F32)
    gg_launch(act_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)in, (float*)out, (size_t)n, kind);
  else if (act_dtype == GG_BF16)
    gg_launch(act_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in,
              (__nv_bfloat16*)out, (size_t)n, kind);
  else
    return gg_fail(GG_ERR_INVALID, "act: unknown dtype %d", act_dtype);
  return gg_check_launch("act");
}
