// A state-space layer of the Mamba-2 kind around the linear recurrence of delta_rule.cu.  Per head
// (P values, a state S [N, P] in float32 carried in the request's state slot):
//     S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x
// with x (H heads of P values), B and C (G groups of N values; head h reads group h / (H / G)) passed
// through a short causal convolution per channel (with bias) and SiLU, dt = softplus(dt + dt_bias)
// per head.  The result is multiplied by silu(z) and RMS-normed in equal parts of the row.
//
// Kernels of a step (any mix of prompt portions and single decoded tokens):
//   ssm_prep   per (token, 128 channels): convolution + bias + SiLU from the projection's columns
//              [z | x | B | C | dt] and the window carried in the state slot; written as float32 rows
//              [C | B | x], the order the recurrence kernel reads (q, k, v); the last block of a token
//              computes the step size and the decay.  Then the window is moved on.
//   (the recurrence: gg_delta_recur with plain = 1: k = B, q = C, v = x, beta = dt)
//   ssm_out    per (token, part): (y + D x) * silu(z), divided by the part's root mean square, times
//              the weight
// Everything here is float32 arithmetic; the projection that comes in and the result that goes out
// are in the activation type.
#include "common.cuh"

int conv_state_update(const void* x, long long x_stride, int dtype, float* conv_state, const int* cu_q_lens,
                      const int* context_lens, const int* state_slots, int B, int C, int taps, cudaStream_t stream);

__device__ __forceinline__ int ssm_seq_of_token(const int* __restrict__ cu, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}
__device__ __forceinline__ float ssm_silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float ssm_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

#define SSM_CH 128

// grid (T, ceil(Cc / 128) + 1).  proj [T, stride]: [z: inner | x: inner | B: G*N | C: G*N | dt: H];
// conv_w [Cc, taps], conv_b [Cc] over the channels x, B, C (Cc = inner + 2 G N); conv_state
// [slots, taps-1, Cc] holds the inputs at positions start-(taps-1) .. start-1 of the sequence.
template <typename TA>
__global__ void ssm_prep_kernel(const TA* __restrict__ proj, long long stride, const float* __restrict__ conv_w,
                                const float* __restrict__ conv_b, const float* __restrict__ conv_state,
                                const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                                const int* __restrict__ state_slots, int B, int H, int P, int G, int N, int taps,
                                float* __restrict__ cbx, float* __restrict__ dt_out, float* __restrict__ decay) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int inner = H * P, GN = G * N, Cc = inner + 2 * GN;
  const int b = ssm_seq_of_token(cu_q_lens, B, t);
  const int t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  const int slot = state_slots[b];
  const int start = context_lens[b] - qlen;
  pdl_wait();
  if (blockIdx.y == gridDim.y - 1) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float dt = ssm_softplus(to_f32(proj[(size_t)t * stride + 2 * inner + 2 * GN + h]) + dt_bias[h]);
      dt_out[(size_t)t * H + h] = dt;
      decay[(size_t)t * H + h] = expf(-expf(a_log[h]) * dt);
    }
    return;
  }
  const int c = blockIdx.y * SSM_CH + threadIdx.x;
  if (c >= Cc) return;
  const int i = t - t0;
  const float* st = (slot >= 0 && start > 0) ? conv_state + (size_t)slot * (taps - 1) * Cc : nullptr;
  float acc = conv_b ? conv_b[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = i - (taps - 1) + j;
    float xv;
    if (src >= 0) xv = to_f32(proj[(size_t)(t0 + src) * stride + inner + c]);
    else xv = st ? st[(size_t)(taps - 1 + src) * Cc + c] : 0.f;
    acc = fmaf(conv_w[(size_t)c * taps + j], xv, acc);
  }
  // x, B, C -> rows [C | B | x]
  const int dst = c < inner ? 2 * GN + c : (c < inner + GN ? GN + (c - inner) : c - inner - GN);
  cbx[(size_t)t * Cc + dst] = ssm_silu(acc);
}

// grid (T, parts): part p of token t covers inner / parts values.
template <typename TA>
__global__ void ssm_out_kernel(const float* __restrict__ y_raw, const float* __restrict__ cbx, int x_col, int Cc,
                               const TA* __restrict__ z, long long z_stride, const float* __restrict__ D,
                               const float* __restrict__ w, float eps, int P, int part, TA* __restrict__ out, int inner) {
  extern __shared__ float vals[];       // part floats + 33
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c0 = blockIdx.y * part;
  float ss = 0.f;
  for (int e = threadIdx.x; e < part; e += blockDim.x) {
    const int c = c0 + e;
    const float x = cbx[(size_t)t * Cc + x_col + c];
    const float v = (y_raw[(size_t)t * inner + c] + D[c / P] * x) * ssm_silu(to_f32(z[(size_t)t * z_stride + c]));
    vals[e] = v;
    ss += v * v;
  }
  const float f = rsqrtf(block_sum(ss, vals + part) / (float)part + eps);
  for (int e = threadIdx.x; e < part; e += blockDim.x)
    out[(size_t)t * inner + c0 + e] = from_f32<TA>(vals[e] * f * w[c0 + e]);
}

extern "C" int gg_ssm_prep(const void* proj, long long stride, int dtype, const float* conv_w, const float* conv_b,
                           float* conv_state, const float* a_log, const float* dt_bias, const int* cu_q_lens,
                           const int* context_lens, const int* state_slots, int T, int B, int H, int P, int G, int N,
                           int taps, float* cbx, float* dt_out, float* decay, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && B > 0 && H > 0 && P > 0 && G > 0 && N > 0 && H % G == 0, "ssm_prep: bad sizes T=%d B=%d H=%d P=%d G=%d N=%d", T, B, H, P, G, N);
  GG_REQUIRE(taps >= 1 && taps <= 17, "ssm_prep: %d taps are outside 1..17", taps);
  const int inner = H * P, Cc = inner + 2 * G * N;
  GG_REQUIRE(stride >= (long long)inner + Cc + H, "ssm_prep: rows of %lld values are too short", stride);
  GG_REQUIRE(taps == 1 || conv_state, "ssm_prep: no room for the convolution's window");
  if (T == 0) return GG_OK;
  const dim3 grid(T, (Cc + SSM_CH - 1) / SSM_CH + 1);
  GG_REQUIRE(grid.y <= 65535, "ssm_prep: too many channels");
  if (dtype == GG_F32)
    gg_launch(ssm_prep_kernel<float>, grid, dim3(SSM_CH), 0, stream, (const float*)proj, stride, conv_w, conv_b, (const float*)conv_state, a_log, dt_bias, cu_q_lens, context_lens, state_slots, B, H, P, G, N, taps, cbx, dt_out, decay);
  else if (dtype == GG_BF16)
    gg_launch(ssm_prep_kernel<__nv_bfloat16>, grid, dim3(SSM_CH), 0, stream, (const __nv_bfloat16*)proj, stride, conv_w, conv_b, (const float*)conv_state, a_log, dt_bias, cu_q_lens, context_lens, state_slots, B, H, P, G, N, taps, cbx, dt_out, decay);
  else
    return gg_fail(GG_ERR_INVALID, "ssm_prep: unknown dtype %d", dtype);
  int rc = gg_check_launch("ssm_prep");
  if (rc || taps == 1) return rc;
  const size_t esize = dtype == GG_F32 ? 4 : 2;
  return conv_state_update((const char*)proj + (size_t)inner * esize, stride, dtype, conv_state, cu_q_lens, context_lens,
                           state_slots, B, Cc, taps, stream);
}

extern "C" int gg_ssm_out(const float* y_raw, const float* cbx, int x_col, int Cc, const void* z, long long z_stride,
                          int dtype, const float* D, const float* w, float eps, int T, int H, int P, int parts, void* out,
                          cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && P > 0 && parts > 0 && (H * P) % parts == 0 && parts <= 65535, "ssm_out: bad sizes T=%d H=%d P=%d parts=%d", T, H, P, parts);
  if (T == 0) return GG_OK;
  const int inner = H * P, part = inner / parts;
  const size_t smem = (size_t)(part + 33) * sizeof(float);
  GG_REQUIRE(smem <= 200 * 1024, "ssm_out: parts of %d values do not fit in shared memory", part);
  // four values a thread where the part is long: a step of few decoded tokens has T * parts blocks and waits on
  // each thread's chain of reads
  const int threads = part >= 4096 ? 1024 : (part >= 2048 ? 512 : (part >= 1024 ? 256 : (part >= 256 ? 128 : 64)));
  const dim3 grid(T, parts);
  cudaError_t e = cudaSuccess;
  if (dtype == GG_F32) {
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(ssm_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "ssm_out: %s", cudaGetErrorString(e));
    gg_launch(ssm_out_kernel<float>, grid, dim3(threads), smem, stream, y_raw, cbx, x_col, Cc, (const float*)z, z_stride, D, w, eps, P, part, (float*)out, inner);
  } else if (dtype == GG_BF16) {
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(ssm_out_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "ssm_out: %s", cudaGetErrorString(e));
    gg_launch(ssm_out_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, y_raw, cbx, x_col, Cc, (const __nv_bfloat16*)z, z_stride, D, w, eps, P, part, (__nv_bfloat16*)out, inner);
  } else
    return gg_fail(GG_ERR_INVALID, "ssm_out: unknown dtype %d", dtype);
  return gg_check_launch("ssm_out");
}
