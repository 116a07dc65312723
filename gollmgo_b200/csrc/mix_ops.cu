// Small per-row kernels that join the branches of a layer: the weighted sum of RMS-normed
// branch outputs, the scaled add of sublayer outputs to the residual stream, a bias on rows,
// the rounded concatenation of two float32 streams, a clamped gated activation, and the
// combination of the two maps of a differential attention.  Float32 arithmetic throughout.
#include "common.cuh"

#define MIX_MAX 4

struct MixArgs {
  const void* y[MIX_MAX];       // [T, W] each, activation type
  const float* w[MIX_MAX];      // [W] each
  int n;
};

// out[t, :] = coef * sum_i  y_i[t, :] / sqrt(mean(y_i[t, :]^2) + eps) * w_i
template <typename TA>
__global__ void rms_mix_kernel(MixArgs m, float coef, float eps, int W, TA* __restrict__ out) {
  __shared__ float red[33];
  __shared__ float f[MIX_MAX];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = 0; i < m.n; ++i) {
    const TA* y = (const TA*)m.y[i] + (size_t)t * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = to_f32(y[c]); ss += v * v; }
    const float tot = block_sum(ss, red);
    if (threadIdx.x == 0) f[i] = rsqrtf(tot / (float)W + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < m.n; ++i) acc += to_f32(((const TA*)m.y[i])[(size_t)t * W + c]) * f[i] * m.w[i][c];
    out[(size_t)t * W + c] = from_f32<TA>(coef * acc);
  }
}

extern "C" int gg_rms_mix(const void* const* ys, const float* const* ws, int n, float coef, float eps, int T, int W,
                          int dtype, void* out, cudaStream_t stream) {
  GG_REQUIRE(n >= 1 && n <= MIX_MAX, "rms_mix: %d branches are outside 1..%d", n, MIX_MAX);
  GG_REQUIRE(T >= 0 && W > 0, "rms_mix: bad sizes T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  MixArgs m = {};
  m.n = n;
  for (int i = 0; i < n; ++i) { m.y[i] = ys[i]; m.w[i] = ws[i]; }
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == GG_F32) gg_launch(rms_mix_kernel<float>, dim3(T), dim3(threads), 0, stream, m, coef, eps, W, (float*)out);
  else if (dtype == GG_BF16) gg_launch(rms_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, m, coef, eps, W, (__nv_bfloat16*)out);
  else return gg_fail(GG_ERR_INVALID, "rms_mix: unknown dtype %d", dtype);
  return gg_check_launch("rms_mix");
}

// resid[i] += mult * (a[i] + b[i] + bias[i % W])          b, bias optional
template <typename TA>
__global__ void scaled_add_kernel(float* __restrict__ resid, const TA* __restrict__ a, const TA* __restrict__ b,
                                  const float* __restrict__ bias, float mult, long long n, int W) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = to_f32(a[i]);
    if (b) v += to_f32(b[i]);
    if (bias) v += bias[i % W];
    resid[i] += mult * v;
  }
}

extern "C" int gg_scaled_add(float* resid, const void* a, const void* b, const float* bias, float mult, int T, int W,
                             int dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0 && a, "scaled_add: bad sizes T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(scaled_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, resid, (const float*)a, (const float*)b, bias, mult, n, W);
  else if (dtype == GG_BF16) gg_launch(scaled_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, resid, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, bias, mult, n, W);
  else return gg_fail(GG_ERR_INVALID, "scaled_add: unknown dtype %d", dtype);
  return gg_check_launch("scaled_add");
}

// y[t, c] += bias[c]
template <typename TA>
__global__ void bias_add_kernel(TA* __restrict__ y, const float* __restrict__ bias, long long n, int W) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = from_f32<TA>(to_f32(y[i]) + bias[i % W]);
}

extern "C" int gg_bias_add(void* y, const float* bias, int T, int W, int dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0 && bias, "bias_add: bad sizes T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(bias_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)y, bias, n, W);
  else if (dtype == GG_BF16) gg_launch(bias_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)y, bias, n, W);
  else return gg_fail(GG_ERR_INVALID, "bias_add: unknown dtype %d", dtype);
  return gg_check_launch("bias_add");
}

// out[t, :] = [a[t, :] (+ da[t, :]), b[t, :]] rounded to the activation type; a, b float32 [T, W]
template <typename TA>
__global__ void concat_cast_kernel(const float* __restrict__ a, const TA* __restrict__ da, const float* __restrict__ b,
                                   TA* __restrict__ out, long long n, int W) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / W;
    const int c = (int)(i - t * W);
    out[t * 2 * W + c] = from_f32<TA>(a[i] + (da ? to_f32(da[i]) : 0.f));
    out[t * 2 * W + W + c] = from_f32<TA>(b[i]);
  }
}

extern "C" int gg_concat_cast(const float* a, const void* da, const float* b, void* out, int T, int W, int dtype,
                              cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0, "concat_cast: bad sizes T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(concat_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, (const float*)da, b, (float*)out, n, W);
  else if (dtype == GG_BF16) gg_launch(concat_cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, a, (const __nv_bfloat16*)da, b, (__nv_bfloat16*)out, n, W);
  else return gg_fail(GG_ERR_INVALID, "concat_cast: unknown dtype %d", dtype);
  return gg_check_launch("concat_cast");
}

// Clamped gated activation on [T, 2I] -> [T, I]:
//   g = min(gate, limit); u = clamp(up, -limit, limit); out = g * sigmoid(alpha * g) * (u + shift)
__device__ __forceinline__ float clamped_gate_f(float gate, float up, float limit, float alpha, float shift) {
  const float g = fminf(gate, limit);
  const float u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + shift);
}

template <typename TA>
__global__ void clamped_gate_kernel(const TA* __restrict__ gu, TA* __restrict__ out, long long n, int I, float limit,
                                    float alpha, float shift) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / I;
    const int c = (int)(i - t * I);
    out[i] = from_f32<TA>(clamped_gate_f(to_f32(gu[t * 2 * I + c]), to_f32(gu[t * 2 * I + I + c]), limit, alpha, shift));
  }
}

// bfloat16 with I a multiple of 8: eight values a thread, 16-byte loads and stores
__global__ void clamped_gate_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long n8,
                                        int I8, float limit, float alpha, float shift) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / I8;
    const int c = (int)(i - t * I8);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + c) * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + c) * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(clamped_gate_f(g.x, u.x, limit, alpha, shift), clamped_gate_f(g.y, u.y, limit, alpha, shift));
    }
    *reinterpret_cast<uint4*>(out + i * 8) = o4;
  }
}

extern "C" int gg_clamped_gate(const void* gu, void* out, int T, int I, float limit, float alpha, float shift, int dtype,
                               cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && I > 0, "clamped_gate: bad sizes T=%d I=%d", T, I);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * I;
  if (dtype == GG_BF16 && I % 8 == 0 && ((size_t)gu % 16) == 0 && ((size_t)out % 16) == 0) {
    const long long n8 = n / 8;
    const int blocks = (int)((n8 + 255) / 256 < 8192 ? (n8 + 255) / 256 : 8192);
    gg_launch(clamped_gate_vec_kernel, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n8, I / 8, limit, alpha, shift);
    return gg_check_launch("clamped_gate");
  }
  const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
  if (dtype == GG_F32) gg_launch(clamped_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, n, I, limit, alpha, shift);
  else if (dtype == GG_BF16) gg_launch(clamped_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n, I, limit, alpha, shift);
  else return gg_fail(GG_ERR_INVALID, "clamped_gate: unknown dtype %d", dtype);
  return gg_check_launch("clamped_gate");
}

// Differential attention: the two maps of a head, a [T, 2H, dv] float32 with the maps of kv
// group g laid out as [g][map][head in group], are combined as
//   o = a1 - lambda * a2;  out[t, h, :] = o / sqrt(mean(o^2) + eps) * post
// grid (T, H).
template <typename TA>
__global__ void diff_combine_kernel(const float* __restrict__ a, TA* __restrict__ out, float lambda, float eps,
                                    float post, int H, int G, int dv) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, rep = H / G, g = h / rep, j = h - g * rep;
  const float* a1 = a + ((size_t)t * 2 * H + (size_t)(g * 2) * rep + j) * dv;
  const float* a2 = a + ((size_t)t * 2 * H + (size_t)(g * 2 + 1) * rep + j) * dv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) { const float o = a1[c] - lambda * a2[c]; ss += o * o; }
  const float f = rsqrtf(block_sum(ss, red) / (float)dv + eps) * post;
  TA* y = out + ((size_t)t * H + h) * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) y[c] = from_f32<TA>((a1[c] - lambda * a2[c]) * f);
}

extern "C" int gg_diff_combine(const float* a, void* out, float lambda, float eps, float post, int T, int H, int G,
                               int dv, int dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dv > 0 && H <= 65535, "diff_combine: bad sizes T=%d H=%d G=%d dv=%d", T, H, G, dv);
  if (T == 0) return GG_OK;
  const int threads = dv >= 256 ? 256 : (dv >= 128 ? 128 : 64);
  const dim3 grid(T, H);
  if (dtype == GG_F32) gg_launch(diff_combine_kernel<float>, grid, dim3(threads), 0, stream, a, (float*)out, lambda, eps, post, H, G, dv);
  else if (dtype == GG_BF16) gg_launch(diff_combine_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, a, (__nv_bfloat16*)out, lambda, eps, post, H, G, dv);
  else return gg_fail(GG_ERR_INVALID, "diff_combine: unknown dtype %d", dtype);
  return gg_check_launch("diff_combine");
}

// ---------------------------------------------------------------- weighted sum of branches
// out[t, :] = sum_i coef_i * y_i[t, :]
struct SumArgs {
  const void* y[MIX_MAX];
  float coef[MIX_MAX];
  int n;
};

template <typename TA>
__global__ void weighted_sum_kernel(SumArgs m, long long n, TA* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int j = 0; j < m.n; ++j) v = fmaf(m.coef[j], to_f32(((const TA*)m.y[j])[i]), v);
    out[i] = from_f32<TA>(v);
  }
}

extern "C" int gg_weighted_sum(const void* const* ys, const float* coefs, int n, int T, int W, int dtype, void* out,
                               cudaStream_t stream) {
  GG_REQUIRE(n >= 1 && n <= MIX_MAX && T >= 0 && W > 0, "weighted_sum: bad sizes n=%d T=%d W=%d", n, T, W);
  if (T == 0) return GG_OK;
  SumArgs m = {};
  m.n = n;
  for (int i = 0; i < n; ++i) { m.y[i] = ys[i]; m.coef[i] = coefs[i]; }
  const long long total = (long long)T * W;
  const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(weighted_sum_kernel<float>, dim3(blocks), dim3(256), 0, stream, m, total, (float*)out);
  else if (dtype == GG_BF16) gg_launch(weighted_sum_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, m, total, (__nv_bfloat16*)out);
  else return gg_fail(GG_ERR_INVALID, "weighted_sum: unknown dtype %d", dtype);
  return gg_check_launch("weighted_sum");
}

// ---------------------------------------------------------------- token shift
// out[t] = h[t] + (h[t - 1] - h[t]) * mu, the row before the first token of a step's portion taken
// from the request's state slot (zeros at the start of the sequence); afterwards the slot holds the
// portion's last row.  grid (T): only the block of a portion's first row touches the slot, and every
// thread reads its columns of it before it writes them.
template <typename TA>
__global__ void token_shift_kernel(const TA* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                                   const int* __restrict__ state_slots, int B, int W, TA* __restrict__ out) {
  pdl_trigger();
  const int t = blockIdx.x;
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q_lens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int b = lo, t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  const int slot = state_slots[b];
  const int start = context_lens[b] - qlen;
  pdl_wait();
  const TA* cur = h + (size_t)t * W;
  TA* o = out + (size_t)t * W;
  if (t > t0) {
    const TA* prev = cur - W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float x = to_f32(cur[c]);
      o[c] = from_f32<TA>(fmaf(to_f32(prev[c]) - x, mu[c], x));
    }
    return;
  }
  float* st = slot >= 0 ? state + (size_t)slot * W : nullptr;
  const TA* last = h + (size_t)(t0 + qlen - 1) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float x = to_f32(cur[c]);
    const float p = (st && start > 0) ? st[c] : 0.f;
    o[c] = from_f32<TA>(fmaf(p - x, mu[c], x));
    if (st) st[c] = to_f32(last[c]);
  }
}

extern "C" int gg_token_shift(const void* h, const float* mu, float* state, const int* cu_q_lens, const int* context_lens,
                              const int* state_slots, int T, int B, int W, int dtype, void* out, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && B > 0 && W > 0 && h && mu && state && out, "token_shift: bad arguments T=%d B=%d W=%d", T, B, W);
  if (T == 0) return GG_OK;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == GG_F32) gg_launch(token_shift_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)h, mu, state, cu_q_lens, context_lens, state_slots, B, W, (float*)out);
  else if (dtype == GG_BF16) gg_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)h, mu, state, cu_q_lens, context_lens, state_slots, B, W, (__nv_bfloat16*)out);
  else return gg_fail(GG_ERR_INVALID, "token_shift: unknown dtype %d", dtype);
  return gg_check_launch("token_shift");
}

// ---------------------------------------------------------------- capped logits
// x <- cap * tanh(x / cap), float32, in place
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap, float inv) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

extern "C" int gg_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && cap > 0.f && x, "softcap: bad arguments n=%lld cap=%g", n, (double)cap);
  if (n == 0) return GG_OK;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  gg_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, n, cap, 1.f / cap);
  return gg_check_launch("softcap");
}

// ---------------------------------------------------------------- scaled embedding + learned positions
// resid[t, :] = resid[t, :] * scale + table[positions[t], :]; a position past the table sets the flag
template <typename TA>
__global__ void scale_add_rows_kernel(float* __restrict__ resid, float scale, const TA* __restrict__ table,
                                      const int* __restrict__ positions, int W, int rows, int* __restrict__ bad) {
  pdl_trigger();
  const int t = blockIdx.x;
  int p = positions[t];
  pdl_wait();
  if (p < 0 || p >= rows) {
    if (bad && threadIdx.x == 0) *bad = 1;
    p = p < 0 ? 0 : rows - 1;
  }
  float* x = resid + (size_t)t * W;
  const TA* r = table + (size_t)p * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) x[c] = fmaf(x[c], scale, to_f32(r[c]));
}

extern "C" int gg_scale_add_rows(float* resid, float scale, const void* table, const int* positions, int T, int W,
                                 int rows, int dtype, int* bad, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0 && rows > 0 && resid && table && positions, "scale_add_rows: bad arguments T=%d W=%d rows=%d", T, W, rows);
  if (T == 0) return GG_OK;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == GG_F32) gg_launch(scale_add_rows_kernel<float>, dim3(T), dim3(threads), 0, stream, resid, scale, (const float*)table, positions, W, rows, bad);
  else if (dtype == GG_BF16) gg_launch(scale_add_rows_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, resid, scale, (const __nv_bfloat16*)table, positions, W, rows, bad);
  else return gg_fail(GG_ERR_INVALID, "scale_add_rows: unknown dtype %d", dtype);
  return gg_check_launch("scale_add_rows");
}

// ---------------------------------------------------------------- elementwise sigmoid gate
// out[t, c] = a[t, c] * sigmoid(g[t, c]); a float32 [T, W], g rows of stride g_stride in the activation type
template <typename TA>
__global__ void sigmoid_gate_kernel(const float* __restrict__ a, const TA* __restrict__ g, long long g_stride,
                                    TA* __restrict__ out, long long n, int W) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / W;
    const float z = to_f32(g[t * g_stride + (i - t * W)]);
    out[i] = from_f32<TA>(a[i] / (1.f + expf(-z)));
  }
}

extern "C" int gg_sigmoid_gate(const float* a, const void* g, long long g_stride, void* out, int T, int W, int dtype,
                               cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0 && a && g && out && g_stride >= W, "sigmoid_gate: bad arguments T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, a, (const float*)g, g_stride, (float*)out, n, W);
  else if (dtype == GG_BF16) gg_launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, a, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, n, W);
  else return gg_fail(GG_ERR_INVALID, "sigmoid_gate: unknown dtype %d", dtype);
  return gg_check_launch("sigmoid_gate");
}


// out[t, c] = act(gu[t, c] + bias[c]) * (gu[t, I + c] + bias[I + c]): the inner step of a gated feed-forward whose
// two first products have biases (bias null: none).  kind 0: relu, 1: gelu (tanh form), 2: silu.
__device__ __forceinline__ float gated_act_apply(float z, int kind) {
  if (kind == 0) return fmaxf(z, 0.f);
  if (kind == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

template <typename TA>
__global__ void gated_act_kernel(const TA* __restrict__ gu, const float* __restrict__ bias, TA* __restrict__ out, int I, int kind) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.y;
  const TA* row = gu + t * 2 * I;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < I; c += gridDim.x * blockDim.x) {
    const float g = to_f32(row[c]) + (bias ? bias[c] : 0.f), u = to_f32(row[I + c]) + (bias ? bias[I + c] : 0.f);
    out[t * I + c] = from_f32<TA>(gated_act_apply(g, kind) * u);
  }
}

// 16 bytes of gates and of ups a thread (I a multiple of that many values, rows 16-byte aligned)
template <typename TA>
__global__ void gated_act_vec_kernel(const TA* __restrict__ gu, const float* __restrict__ bias, TA* __restrict__ out, int I, int kind) {
  constexpr int VPT = 16 / (int)sizeof(TA);
  pdl_trigger();
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VPT;
  if (c >= I) return;
  const size_t t = blockIdx.y;
  uint4 gr = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c), ur = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c), r;
  const TA* gv = reinterpret_cast<const TA*>(&gr);
  const TA* uv = reinterpret_cast<const TA*>(&ur);
  TA* rv = reinterpret_cast<TA*>(&r);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const float g = to_f32(gv[j]) + (bias ? bias[c + j] : 0.f), u = to_f32(uv[j]) + (bias ? bias[I + c + j] : 0.f);
    rv[j] = from_f32<TA>(gated_act_apply(g, kind) * u);
  }
  *reinterpret_cast<uint4*>(out + t * I + c) = r;
}

extern "C" int gg_gated_act(const void* gu, const float* bias, void* out, int T, int I, int kind, int dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && I > 0 && gu && out && kind >= 0 && kind <= 2, "gated_act: bad arguments T=%d I=%d kind=%d", T, I, kind);
  if (T == 0) return GG_OK;
  const int vpt = dtype == GG_F32 ? 4 : 8;
  if ((dtype == GG_F32 || dtype == GG_BF16) && I % vpt == 0 && T <= 65535 && ((size_t)gu % 16) == 0 && ((size_t)out % 16) == 0) {
    const dim3 grid((I / vpt + 255) / 256, T);
    if (dtype == GG_F32) gg_launch(gated_act_vec_kernel<float>, grid, dim3(256), 0, stream, (const float*)gu, bias, (float*)out, I, kind);
    else gg_launch(gated_act_vec_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)gu, bias, (__nv_bfloat16*)out, I, kind);
    return gg_check_launch("gated_act");
  }
  int gx = (I + 255) / 256;
  if (gx > 64) gx = 64;
  for (int t0 = 0; t0 < T; t0 += 65535) {
    const int n = T - t0 < 65535 ? T - t0 : 65535;
    const dim3 grid(gx, n);
    if (dtype == GG_F32) gg_launch(gated_act_kernel<float>, grid, dim3(256), 0, stream, (const float*)gu + (size_t)t0 * 2 * I, bias, (float*)out + (size_t)t0 * I, I, kind);
    else if (dtype == GG_BF16) gg_launch(gated_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)gu + (size_t)t0 * 2 * I, bias, (__nv_bfloat16*)out + (size_t)t0 * I, I, kind);
    else return gg_fail(GG_ERR_INVALID, "gated_act: unknown dtype %d", dtype);
  }
  return gg_check_launch("gated_act");
}

// a[t, c] *= sigmoid(g[t, c]) in place; a rows of W values, g rows of stride g_stride, both of the activation type
template <typename TA>
__global__ void gate_mul_kernel(TA* __restrict__ a, const TA* __restrict__ g, long long g_stride, long long n, int W) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / W;
    const float z = to_f32(g[t * g_stride + (i - t * W)]);
    a[i] = from_f32<TA>(to_f32(a[i]) / (1.f + expf(-z)));
  }
}

extern "C" int gg_gate_mul(void* a, const void* g, long long g_stride, int T, int W, int dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && W > 0 && a && g && g_stride >= W, "gate_mul: bad arguments T=%d W=%d", T, W);
  if (T == 0) return GG_OK;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  if (dtype == GG_F32) gg_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)a, (const float*)g, g_stride, n, W);
  else if (dtype == GG_BF16) gg_launch(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)a, (const __nv_bfloat16*)g, g_stride, n, W);
  else return gg_fail(GG_ERR_INVALID, "gate_mul: unknown dtype %d", dtype);
  return gg_check_launch("gate_mul");
}
