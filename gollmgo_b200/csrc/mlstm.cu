// The matrix memory with exponential gates (mLSTM) around the engine's plain linear recurrence.
//
// Per head, with log input gate i_t, log forget gate f_t and a running maximum m (m_0 = 0):
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)
// With one more value column that is always 1, n is a column of S: the recurrence kernel of
// csrc/delta_rule.cu (its plain form S <- g S + k (beta v)^T, o = S^T q) then carries both, with
// g = exp(f + m_{t-1} - m_t) and beta = exp(i - m_t).
//
// gg_mlstm_gates: i = cap tanh((zi + bi) / cap), f = logsigmoid(cap tanh((zf + bf) / cap)) (cap <= 0: no
//   cap), the maxima m_t of every sequence's tokens of the step from the m its state slot holds
//   (a block per (sequence, head): the map m -> max(i, f + m) composes, so a warp's 32 tokens are one scan),
//   beta, g and m_t per token, and the new m into the slot.
// gg_mlstm_rows: rows [q | k | v] of the projection (activation type) to float32 rows
//   [q * qscale | k | v, 1, 0..] with the value heads padded to dvp columns.
// gg_mlstm_out: o / (max(|o[dv]|, exp(-m)) + floor), each head divided by its root mean square, times
//   a weight, times sigmoid(gate).
// Everything here is float32 but the projection rows that come in and the gated rows that go out.
#include "common.cuh"

__device__ __forceinline__ float mlstm_cap(float z, float cap) { return cap > 0.f ? cap * tanhf(z / cap) : z; }
__device__ __forceinline__ float mlstm_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// grid (B, H), 32 * NW threads: a warp scans 32 tokens, the block's warps 32 * NW tokens at a time; what a warp's
// tokens do to m together (its last lane's composed map) goes through shared memory, and every warp folds the maps
// of the warps before it over the maximum carried in
__global__ void __launch_bounds__(1024)
mlstm_gates_kernel(const float* __restrict__ zi, long long zi_stride, const float* __restrict__ zf, long long zf_stride,
                   const float* __restrict__ bi, const float* __restrict__ bf, float cap, float* __restrict__ m_state,
                   const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                   const int* __restrict__ state_slots, int H, float* __restrict__ beta, float* __restrict__ decay,
                   float* __restrict__ m_out) {
  __shared__ float aggA[32], aggB[32];
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, NW = blockDim.x >> 5;
  const int slot = state_slots[b];
  const int t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  pdl_wait();
  if (slot < 0 || qlen <= 0) return;
  const int start = context_lens[b] - qlen;
  float carry = start > 0 ? m_state[(size_t)slot * H + h] : 0.f;        // a new sequence starts from m = 0
  const float bih = bi ? bi[h] : 0.f, bfh = bf ? bf[h] : 0.f;
  for (int p0 = 0; p0 < qlen; p0 += 32 * NW) {
    const int tt = p0 + warp * 32 + lane;
    const bool live = tt < qlen;
    float gi = 0.f, gf = 0.f;
    if (live) {
      gi = mlstm_cap(zi[(size_t)(t0 + tt) * zi_stride + h] + bih, cap);
      gf = mlstm_logsigmoid(mlstm_cap(zf[(size_t)(t0 + tt) * zf_stride + h] + bfh, cap));
    }
    // the token's map m -> max(B, A + m); lanes past the end hold the identity (A = 0, B = -inf)
    float A = live ? gf : 0.f, Bm = live ? gi : -INFINITY;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Ae = __shfl_up_sync(0xffffffffu, A, o), Be = __shfl_up_sync(0xffffffffu, Bm, o);
      if (lane >= o) { Bm = fmaxf(Bm, A + Be); A += Ae; }
    }
    if (lane == 31) { aggA[warp] = A; aggB[warp] = Bm; }
    __syncthreads();
    float m_in = carry;
    for (int j = 0; j < warp; ++j) m_in = fmaxf(aggB[j], aggA[j] + m_in);
    const float m = fmaxf(Bm, A + m_in);
    float prev = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) prev = m_in;
    if (live) {
      const size_t at = (size_t)(t0 + tt) * H + h;
      beta[at] = expf(gi - m);
      decay[at] = expf(gf + prev - m);
      m_out[at] = m;
    }
    for (int j = 0; j < NW; ++j) carry = fmaxf(aggB[j], aggA[j] + carry);
    __syncthreads();
  }
  if (threadIdx.x == 0) m_state[(size_t)slot * H + h] = carry;
}

// grid (T, ceil(C / 1024)), 256 threads, four values a thread: out row = [q * qscale (H*d) | k (H*d) | per head: v (dv), 1,
// zeros up to dvp], C its length
template <typename TA>
__global__ void mlstm_rows_kernel(const TA* __restrict__ x, long long x_stride, int H, int d, int dv, int dvp,
                                  float qscale, float* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int qk = H * d, C = 2 * qk + H * dvp;
  const TA* xr = x + t * x_stride;
  float* o = out + t * C;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = blockIdx.y * 1024 + k * 256 + threadIdx.x;
    if (c >= C) break;
    if (c < 2 * qk) {
      o[c] = to_f32(xr[c]) * (c < qk ? qscale : 1.f);
    } else {
      const int e = c - 2 * qk, h = e / dvp, j = e - h * dvp;
      o[c] = j < dv ? to_f32(xr[2 * qk + h * dv + j]) : (j == dv ? 1.f : 0.f);
    }
  }
}

// grid (T, H), 128 threads
template <typename TA>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ m_row, const TA* __restrict__ gate,
                 long long gate_stride, const float* __restrict__ w, float eps, float floor_, int H, int dv, int dvp,
                 TA* __restrict__ out) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int h = blockIdx.y;
  const float* o = o_raw + (t * H + h) * dvp;
  const float den = fmaxf(fabsf(o[dv]), expf(-m_row[t * H + h])) + floor_;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) { const float y = o[c] / den; ss += y * y; }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)dv + eps);
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    const float z = to_f32(gate[t * gate_stride + h * dv + c]);
    out[(t * H + h) * dv + c] = from_f32<TA>(o[c] / den * rinv * w[h * dv + c] / (1.f + expf(-z)));
  }
}

extern "C" int gg_mlstm_gates(const float* zi, long long zi_stride, const float* zf, long long zf_stride, const float* bi,
                              const float* bf, float cap, float* m_state, const int* cu_q_lens, const int* context_lens,
                              const int* state_slots, int B, int H, int T, float* beta, float* decay, float* m_out,
                              cudaStream_t stream) {
  GG_REQUIRE(B > 0 && H > 0 && zi && zf && m_state && beta && decay && m_out, "mlstm_gates: bad arguments B=%d H=%d", B, H);
  GG_REQUIRE(zi_stride >= H && zf_stride >= H, "mlstm_gates: gate rows shorter than %d heads", H);
  GG_REQUIRE(H <= 65535 && T >= 0, "mlstm_gates: too many heads");
  const int warps = T > 4 * B ? 16 : 1;          // a step with prompt portions: 512 tokens of a sequence at a time
  gg_launch(mlstm_gates_kernel, dim3(B, H), dim3(32 * warps), 0, stream, zi, zi_stride, zf, zf_stride, bi, bf, cap, m_state,
            cu_q_lens, context_lens, state_slots, H, beta, decay, m_out);
  return gg_check_launch("mlstm_gates");
}

extern "C" int gg_mlstm_rows(const void* x, long long x_stride, int dtype, int T, int H, int d, int dv, int dvp, float qscale,
                             float* out, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && d > 0 && dv > 0 && dvp > dv, "mlstm_rows: bad sizes T=%d H=%d d=%d dv=%d dvp=%d", T, H, d, dv, dvp);
  GG_REQUIRE(x && out && x_stride >= (long long)H * (2 * d + dv), "mlstm_rows: rows of %lld values are too short", x_stride);
  if (T == 0) return GG_OK;
  const int C = H * (2 * d + dvp);
  GG_REQUIRE((C + 1023) / 1024 <= 65535, "mlstm_rows: rows of %d values are too long", C);
  if (dtype == GG_F32) gg_launch(mlstm_rows_kernel<float>, dim3(T, (C + 1023) / 1024), dim3(256), 0, stream, (const float*)x, x_stride, H, d, dv, dvp, qscale, out);
  else if (dtype == GG_BF16) gg_launch(mlstm_rows_kernel<__nv_bfloat16>, dim3(T, (C + 1023) / 1024), dim3(256), 0, stream, (const __nv_bfloat16*)x, x_stride, H, d, dv, dvp, qscale, out);
  else return gg_fail(GG_ERR_INVALID, "mlstm_rows: unknown dtype %d", dtype);
  return gg_check_launch("mlstm_rows");
}

extern "C" int gg_mlstm_out(const float* o_raw, const float* m_row, const void* gate, long long gate_stride, int dtype,
                            const float* w, float eps, float floor_, int T, int H, int dv, int dvp, void* out,
                            cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && H <= 65535 && dv > 0 && dvp > dv, "mlstm_out: bad sizes T=%d H=%d dv=%d dvp=%d", T, H, dv, dvp);
  GG_REQUIRE(o_raw && m_row && gate && w && out && gate_stride >= (long long)H * dv, "mlstm_out: bad arguments");
  if (T == 0) return GG_OK;
  if (dtype == GG_F32) gg_launch(mlstm_out_kernel<float>, dim3(T, H), dim3(128), 0, stream, o_raw, m_row, (const float*)gate, gate_stride, w, eps, floor_, H, dv, dvp, (float*)out);
  else if (dtype == GG_BF16) gg_launch(mlstm_out_kernel<__nv_bfloat16>, dim3(T, H), dim3(128), 0, stream, o_raw, m_row, (const __nv_bfloat16*)gate, gate_stride, w, eps, floor_, H, dv, dvp, (__nv_bfloat16*)out);
  else return gg_fail(GG_ERR_INVALID, "mlstm_out: unknown dtype %d", dtype);
  return gg_check_launch("mlstm_out");
}
