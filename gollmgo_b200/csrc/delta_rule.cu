// The gated delta rule: a linear-attention layer whose state per head is a matrix S [d, dv] in
// float32, carried from token to token in the request's state slot:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with k, q unit vectors (q also times d^-1/2), beta in (0, 1) and the decay g in (0, 1) per
// head and token.  q, k and v first pass a short causal convolution over time per channel and
// SiLU; the last taps - 1 inputs of every channel are state too.
//
// Three kernels a step, every one for any mix of prompt portions and single decoded tokens:
//   delta_prep     per (token, head unit): convolution + SiLU, unit norms, beta and decay
//   delta_recur    per (sequence, head, 16 value columns): the recurrence over the portion
//   delta_out      per (token, head): o / rms(o) * weight * silu(gate)  (or sigmoid(gate))
// The decay is one number per head and token, or one per head, token and key channel (a row of S).
// and delta_conv_state, which moves the convolution's window on after delta_prep has read it.
// Every column j of S evolves on its own (S[:, j] only ever meets v_j and u_j), so the columns
// of a head are spread over CTAs; eight lanes share a column and split its d rows.
// Everything here is float32 arithmetic; only the projections that come in (x, gate) and the
// result that goes out are in the activation type.
#include "common.cuh"

// Index of the sequence that token t belongs to: the largest b with cu[b] <= t.
__device__ __forceinline__ int seq_of_token(const int* __restrict__ cu, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------- convolution, norms, gates
// grid (T, G + G + H + 1), the last unit of a token computes beta and the decay.
// x [T, x_stride]: columns [q: G*d | k: G*d | v: H*dv]; conv_w [C, taps]; conv_state
// [slots, taps-1, C] holds the inputs at positions start-(taps-1) .. start-1 of the sequence.
template <typename TA>
__global__ void delta_prep_kernel(const TA* __restrict__ x, long long x_stride, const float* __restrict__ conv_w,
                                  const float* __restrict__ conv_state, const float* __restrict__ zb_in, long long zb_stride,
                                  const float* __restrict__ za_in, long long za_stride, int dw,
                                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                  const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                                  const int* __restrict__ state_slots, int B, int G, int H, int d, int dv, int taps,
                                  float* __restrict__ qkv_out, float* __restrict__ beta, float* __restrict__ decay) {
  extern __shared__ float ys[];          // the unit's channels + 33 for the reduction
  pdl_trigger();
  const int t = blockIdx.x, u = blockIdx.y;
  const int C = 2 * G * d + H * dv;
  const int b = seq_of_token(cu_q_lens, B, t);
  const int t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  const int slot = state_slots[b];
  const int start = context_lens[b] - qlen;            // tokens of the sequence before this step
  pdl_wait();
  if (u == 2 * G + H) {
    // dw = 1: one decay per head; dw = d: one per head and key channel
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      beta[(size_t)t * H + h] = 1.f / (1.f + expf(-zb_in[(size_t)t * zb_stride + h]));
    for (int e = threadIdx.x; e < H * dw; e += blockDim.x)
      decay[(size_t)t * H * dw + e] = expf(-expf(a_log[e / dw]) * softplus_f(za_in[(size_t)t * za_stride + e] + dt_bias[e]));
    return;
  }
  const bool unit = u < 2 * G;                           // a q or k head: made a unit vector
  const int dh = unit ? d : dv;
  const int c0 = unit ? u * d : 2 * G * d + (u - 2 * G) * dv;
  const int i = t - t0;                                  // place in the portion
  const float* st = (slot >= 0 && start > 0) ? conv_state + (size_t)slot * (taps - 1) * C : nullptr;
  float ss = 0.f;
  for (int e = threadIdx.x; e < dh; e += blockDim.x) {
    const int c = c0 + e;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = i - (taps - 1) + j;
      float xv;
      if (src >= 0) xv = to_f32(x[(size_t)(t0 + src) * x_stride + c]);
      else xv = st ? st[(size_t)(taps - 1 + src) * C + c] : 0.f;
      acc = fmaf(conv_w[(size_t)c * taps + j], xv, acc);
    }
    const float y = silu_f(acc);
    ys[e] = y;
    ss += y * y;
  }
  float f = 1.f;
  if (unit) {
    const float tot = block_sum(ss, ys + dh);
    f = rsqrtf(tot + 1e-6f);
    if (u < G) f *= rsqrtf((float)d);
  }
  for (int e = threadIdx.x; e < dh; e += blockDim.x) qkv_out[(size_t)t * C + c0 + e] = ys[e] * f;
}

// grid (B, ceil(C / 128)): the window of the convolution after this step's tokens.
template <typename TA>
__global__ void delta_conv_state_kernel(const TA* __restrict__ x, long long x_stride, float* __restrict__ conv_state,
                                        const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                                        const int* __restrict__ state_slots, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = state_slots[b];
  const int t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  if (slot < 0 || qlen <= 0 || c >= C) return;
  const int start = context_lens[b] - qlen;
  float* st = conv_state + (size_t)slot * (taps - 1) * C;
  float keep[16];
#pragma unroll
  for (int s = 0; s < 16; ++s) {
    if (s < taps - 1) {
      const int src = qlen - (taps - 1) + s;
      if (src >= 0) keep[s] = to_f32(x[(size_t)(t0 + src) * x_stride + c]);
      else keep[s] = start > 0 ? st[(size_t)(taps - 1 + src) * C + c] : 0.f;
    }
  }
#pragma unroll
  for (int s = 0; s < 16; ++s)
    if (s < taps - 1) st[(size_t)s * C + c] = keep[s];
}

// ---------------------------------------------------------------- the recurrence
#define DR_COLS 16          // value columns of one CTA
#define DR_LANES 8          // lanes that share a column and split its d rows (dr_row)
#define DR_CHUNK 16         // tokens staged in shared memory at a time
#define DR_STAGE_FLOATS(dp, nc) (2 * DR_CHUNK * (dp) + DR_CHUNK * DR_COLS * (nc) + 2 * DR_CHUNK)
// with a decay per key channel a stage also holds the decays [CHUNK][dp]
#define DR_STAGE_FLOATS_X(dp, ch, nc) (DR_STAGE_FLOATS(dp, nc) + ((ch) ? DR_CHUNK * (dp) : 0))

__device__ __forceinline__ void dr_cp16(float* dst, const float* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Two float32 multiply-adds in one instruction (sm_100: fma.rn.f32x2 and mul.f32x2 on register
// pairs, each half rounded as the scalar instruction rounds).  The recurrence keeps neighbouring
// rows of S as such pairs, which halves the instructions of its inner loop.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}

// Which row of its column lane r holds in register i: four neighbouring rows at a time where there are
// that many (one 16-byte read of shared memory brings a lane four rows of k, q or the decays, and the
// lanes of a column together read 128 neighbouring bytes), else rows r, r + 8.
template <int DPT> __device__ __forceinline__ int dr_row(int i, int r) {
  return DPT >= 4 ? ((i >> 2) * (4 * DR_LANES) + r * 4 + (i & 3)) : (i * DR_LANES + r);
}
// lane r's DPT rows of one token's staged vector [dp]
template <int DPT> __device__ __forceinline__ void dr_rows(float* dst, const float* src, int r) {
  if constexpr (DPT >= 4) {
#pragma unroll
    for (int j = 0; j < DPT / 4; ++j) {
      const float4 v = *reinterpret_cast<const float4*>(src + j * (4 * DR_LANES) + r * 4);
      dst[4 * j] = v.x; dst[4 * j + 1] = v.y; dst[4 * j + 2] = v.z; dst[4 * j + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < DPT; ++i) dst[i] = src[i * DR_LANES + r];
  }
}

// grid (B, H, ceil(dv / (16 NC))), 128 threads.  state [slots, H, dv, d].  NC: columns a thread holds
// (its rows of columns cl, cl + 16, ..): what it reads of k and q from shared memory then serves NC
// columns, which is what bounds the plain recurrence (no chain from token to token but the decay).  CH: decay is [T, H, d], one
// factor per row of S (key channel), and acts before the token's read and write: S <- diag(g) S.
// DELTA = false: the plain linear recurrence S <- g S + k (beta v)^T; o = S^T q (a state-space layer:
// k = B, q = C, v = x, beta = the step size): the token's write does not look at what S holds.
template <int DPT, bool CH, bool DELTA, int NC>
__global__ void __launch_bounds__(DR_COLS * DR_LANES)
delta_recur_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                   float* __restrict__ state, const int* __restrict__ cu_q_lens, const int* __restrict__ context_lens,
                   const int* __restrict__ state_slots, int G, int H, int d, int dv, float* __restrict__ o_raw) {
  extern __shared__ __align__(16) float sm[];
  constexpr int CC = DR_COLS * NC;               // columns of the CTA
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * CC;
  const int tid = threadIdx.x, r = tid & (DR_LANES - 1), cl = tid / DR_LANES;
  const int C = 2 * G * d + H * dv;
  const int slot = state_slots[b];
  const int t0 = cu_q_lens[b], qlen = cu_q_lens[b + 1] - t0;
  if (slot < 0 || qlen <= 0) { pdl_trigger(); return; }
  const int start = context_lens[b] - qlen;
  const int kvh = h / (H / G);
  const int dp = DPT * DR_LANES;                 // d rounded up to what the lanes hold
  float* ks = sm;                                // two stages of k [CHUNK][dp], q [CHUNK][dp], v [CHUNK][COLS], (beta, decay) [CHUNK][2]
  float* os = sm + 2 * DR_STAGE_FLOATS_X(dp, CH, NC);  // [CHUNK][CC][LANES]: every lane's share of o, summed after the chunk
  static_assert(DPT % 2 == 0, "rows are held in pairs");
  constexpr int DP2 = DPT / 2;
  float2 S[NC][DP2];                               // pair p: registers 2p and 2p + 1 of dr_row
  float* shead = state + ((size_t)slot * H + h) * dv * d;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int col = col0 + cl + j * DR_COLS;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int row = dr_row<DPT>(i, r);
      const float v = (col < dv && start > 0 && row < d) ? shead[(size_t)col * d + row] : 0.f;
      if (i & 1) S[j][i >> 1].y = v; else S[j][i >> 1].x = v;
    }
  }
  pdl_wait();
  // A chunk's rows come to shared memory by asynchronous copies, the next chunk's while this one
  // is worked on (plain loads issued in a loop went out one after the other and cost more than
  // the recurrence itself).  16-byte copies where every row starts on such a border.
  const bool vec = (d & 3) == 0 && (dv & 3) == 0;
  auto stage = [&](int c0, int buf) {
    const int n = min(DR_CHUNK, qlen - c0);
    float* kb = ks + buf * DR_STAGE_FLOATS_X(dp, CH, NC);
    float* qb = kb + DR_CHUNK * dp;
    float* vb = qb + DR_CHUNK * dp;
    float* gb = vb + DR_CHUNK * CC;
    float* cb = gb + 2 * DR_CHUNK;                 // CH: the decays of the chunk's tokens
    if (CH) {
      if (vec) {
        const int per = dp >> 2;
        for (int e = tid; e < n * per; e += blockDim.x) {
          const int tt = e / per, row = (e - tt * per) << 2;
          const int bytes = row < d ? 16 : 0;
          dr_cp16(cb + tt * dp + row, decay + ((size_t)(t0 + c0 + tt) * H + h) * d + (bytes ? row : 0), bytes);
        }
      } else {
        for (int e = tid; e < n * dp; e += blockDim.x) {
          const int tt = e / dp, row = e - tt * dp;
          cb[e] = row < d ? decay[((size_t)(t0 + c0 + tt) * H + h) * d + row] : 0.f;
        }
      }
    }
    if (vec) {
      const int per = dp >> 2;
      for (int e = tid; e < n * per; e += blockDim.x) {
        const int tt = e / per, row = (e - tt * per) << 2;
        const float* src = qkv + (size_t)(t0 + c0 + tt) * C;
        const int bytes = row < d ? 16 : 0;
        dr_cp16(kb + tt * dp + row, src + (size_t)(G + kvh) * d + (bytes ? row : 0), bytes);
        dr_cp16(qb + tt * dp + row, src + (size_t)kvh * d + (bytes ? row : 0), bytes);
      }
      for (int e = tid; e < n * (CC / 4); e += blockDim.x) {
        const int tt = e / (CC / 4), cc = (e - tt * (CC / 4)) << 2;
        const int bytes = col0 + cc < dv ? 16 : 0;
        dr_cp16(vb + tt * CC + cc, qkv + (size_t)(t0 + c0 + tt) * C + 2 * G * d + (size_t)h * dv + (bytes ? col0 + cc : 0), bytes);
      }
    } else {
      for (int e = tid; e < n * dp; e += blockDim.x) {
        const int tt = e / dp, row = e - tt * dp;
        const size_t base = (size_t)(t0 + c0 + tt) * C;
        kb[e] = row < d ? qkv[base + (size_t)(G + kvh) * d + row] : 0.f;
        qb[e] = row < d ? qkv[base + (size_t)kvh * d + row] : 0.f;
      }
      for (int e = tid; e < n * CC; e += blockDim.x) {
        const int tt = e / CC, cc = e - tt * CC;
        vb[e] = col0 + cc < dv ? qkv[(size_t)(t0 + c0 + tt) * C + 2 * G * d + (size_t)h * dv + col0 + cc] : 0.f;
      }
    }
    if (tid < n) {
      dr_cp4(gb + tid * 2, beta + (size_t)(t0 + c0 + tid) * H + h);
      if (!CH) dr_cp4(gb + tid * 2 + 1, decay + (size_t)(t0 + c0 + tid) * H + h);
    }
  };
  stage(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int c0 = 0, buf = 0; c0 < qlen; c0 += DR_CHUNK, buf ^= 1) {
    const int n = min(DR_CHUNK, qlen - c0);
    if (c0 + DR_CHUNK < qlen) stage(c0 + DR_CHUNK, buf ^ 1);       // the buffer the chunk before last was read from
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const float* kc = ks + buf * DR_STAGE_FLOATS_X(dp, CH, NC);
    const float* qc = kc + DR_CHUNK * dp;
    const float* vcur = qc + DR_CHUNK * dp;
    const float* bg = vcur + DR_CHUNK * CC;
    const float* gc = bg + 2 * DR_CHUNK;
    // The next token's k, q and decays are read into registers while this token is worked on: the
    // reads of shared memory (which the compiler will not move above the store of the token before)
    // then cost no time on the chain from one token's S to the next.  The sums run in four chains
    // so that the additions overlap.
    constexpr bool PRE = DPT <= 16;                // beyond that the registers would not hold two tokens
    float kn[DPT], qn[DPT], gn[CH ? DPT : 1], vn[NC], ben = 0.f, gdn = 1.f;
    if (PRE) {
      dr_rows<DPT>(kn, kc, r);
      dr_rows<DPT>(qn, qc, r);
      if constexpr (CH) dr_rows<DPT>(gn, gc, r);
#pragma unroll
      for (int j = 0; j < NC; ++j) vn[j] = vcur[cl + j * DR_COLS];
      ben = bg[0];
      if (!CH) gdn = bg[1];
    }
#pragma unroll 2
    for (int tt = 0; tt < n; ++tt) {
      float kv[DPT], qv[DPT], gv[CH ? DPT : 1], vv[NC], be, g = 1.f;
      if (PRE) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) { kv[i] = kn[i]; qv[i] = qn[i]; if constexpr (CH) gv[i] = gn[i]; }
#pragma unroll
        for (int j = 0; j < NC; ++j) vv[j] = vn[j];
        be = ben; g = gdn;
        const int nx = min(tt + 1, n - 1);
        dr_rows<DPT>(kn, kc + nx * dp, r);
        dr_rows<DPT>(qn, qc + nx * dp, r);
        if constexpr (CH) dr_rows<DPT>(gn, gc + nx * dp, r);
#pragma unroll
        for (int j = 0; j < NC; ++j) vn[j] = vcur[nx * CC + cl + j * DR_COLS];
        ben = bg[nx * 2];
        if (!CH) gdn = bg[nx * 2 + 1];
      } else {
        dr_rows<DPT>(kv, kc + tt * dp, r);
        dr_rows<DPT>(qv, qc + tt * dp, r);
        if constexpr (CH) dr_rows<DPT>(gv, gc + tt * dp, r);
#pragma unroll
        for (int j = 0; j < NC; ++j) vv[j] = vcur[tt * CC + cl + j * DR_COLS];
        be = bg[tt * 2];
        if (!CH) g = bg[tt * 2 + 1];
      }
      float2 k2[DP2], q2[DP2], gv2[CH ? DP2 : 1];
#pragma unroll
      for (int p = 0; p < DP2; ++p) {
        k2[p] = make_float2(kv[2 * p], kv[2 * p + 1]);
        q2[p] = make_float2(qv[2 * p], qv[2 * p + 1]);
        if constexpr (CH) gv2[p] = make_float2(gv[2 * p], gv[2 * p + 1]);
      }
      const float2 g2 = make_float2(g, g);
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        float2 d2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int p = 0; p < DP2; ++p) {
          if constexpr (CH) S[j][p] = fmul2(S[j][p], gv2[p]);    // every row by its own factor, first
          if (DELTA) d2[p & 1] = ffma2(k2[p], S[j][p], d2[p & 1]);
        }
        float dot = 0.f;
        if (DELTA) {
          dot = (d2[0].x + d2[0].y) + (d2[1].x + d2[1].y);
          dot += __shfl_xor_sync(0xffffffffu, dot, 1);
          dot += __shfl_xor_sync(0xffffffffu, dot, 2);
          dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        }
        const float u = be * (vv[j] - g * dot);
        const float2 u2 = make_float2(u, u);
        float2 o2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int p = 0; p < DP2; ++p) {
          S[j][p] = ffma2(k2[p], u2, CH ? S[j][p] : fmul2(g2, S[j][p]));
          o2[p & 1] = ffma2(q2[p], S[j][p], o2[p & 1]);
        }
        // the lanes' shares of o are not needed by the next token: they go to shared memory as they are
        // (a store the warp does not wait for), and are summed once the chunk is through
        os[(tt * CC + j * DR_COLS) * DR_LANES + tid] = (o2[0].x + o2[0].y) + (o2[1].x + o2[1].y);
      }
    }
    __syncthreads();
    for (int e = tid; e < n * CC; e += blockDim.x) {
      const int tt = e / CC, cc = e - tt * CC;
      const float4 a = *reinterpret_cast<const float4*>(os + e * DR_LANES), c = *reinterpret_cast<const float4*>(os + e * DR_LANES + 4);
      if (col0 + cc < dv)
        o_raw[(size_t)(t0 + c0 + tt) * H * dv + (size_t)h * dv + col0 + cc] = ((a.x + a.y) + (a.z + a.w)) + ((c.x + c.y) + (c.z + c.w));
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  pdl_trigger();                                 // only now: blocks of the next kernel that wait on a multiprocessor take room there
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int col = col0 + cl + j * DR_COLS;
    if (col < dv) {
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int row = dr_row<DPT>(i, r);
        if (row < d) shead[(size_t)col * d + row] = (i & 1) ? S[j][i >> 1].y : S[j][i >> 1].x;
      }
    }
  }
}

// ---------------------------------------------------------------- the gated norm of the result
// grid (T, H): out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :])
template <typename TA>
__global__ void delta_out_kernel(const float* __restrict__ o_raw, const TA* __restrict__ gate, long long gate_stride,
                                 const float* __restrict__ w, float eps, int H, int dv, int gate_act, TA* __restrict__ out) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* o = o_raw + (size_t)t * H * dv + (size_t)h * dv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) ss += o[c] * o[c];
  const float f = rsqrtf(block_sum(ss, red) / (float)dv + eps);
  const TA* gr = gate + (size_t)t * gate_stride + (size_t)h * dv;
  TA* y = out + (size_t)t * H * dv + (size_t)h * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    const float z = to_f32(gr[c]);
    y[c] = from_f32<TA>(o[c] * f * w[c] * (gate_act == 1 ? 1.f / (1.f + expf(-z)) : silu_f(z)));
  }
}

// ---------------------------------------------------------------- launchers
// The window of a short convolution over the C channels x[:, 0 .. C) moved on by this step's tokens
// (also for the state-space layer, ssm.cu).
int conv_state_update(const void* x, long long x_stride, int dtype, float* conv_state, const int* cu_q_lens,
                      const int* context_lens, const int* state_slots, int B, int C, int taps, cudaStream_t stream) {
  const dim3 sgrid(B, (C + 127) / 128);
  if (dtype == GG_F32)
    gg_launch(delta_conv_state_kernel<float>, sgrid, dim3(128), 0, stream, (const float*)x, x_stride, conv_state, cu_q_lens, context_lens, state_slots, C, taps);
  else
    gg_launch(delta_conv_state_kernel<__nv_bfloat16>, sgrid, dim3(128), 0, stream, (const __nv_bfloat16*)x, x_stride, conv_state, cu_q_lens, context_lens, state_slots, C, taps);
  return gg_check_launch("conv_state_update");
}

extern "C" int gg_delta_prep(const void* x, long long x_stride, int dtype, const float* conv_w, float* conv_state,
                             const float* zb, long long zb_stride, const float* za, long long za_stride, int dw,
                             const float* a_log, const float* dt_bias, const int* cu_q_lens,
                             const int* context_lens, const int* state_slots, int T, int B, int G, int H, int d, int dv,
                             int taps, float* qkv_out, float* beta, float* decay, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && B > 0 && G > 0 && H > 0 && H % G == 0 && d > 0 && dv > 0, "delta_prep: bad sizes T=%d B=%d G=%d H=%d d=%d dv=%d", T, B, G, H, d, dv);
  GG_REQUIRE(taps >= 1 && taps <= 17, "delta_prep: %d taps are outside 1..17", taps);
  GG_REQUIRE(dw == 1 || dw == d, "delta_prep: a decay per head (1) or per key channel (%d), not %d", d, dw);
  GG_REQUIRE(zb && za && zb_stride >= H && za_stride >= (long long)H * dw, "delta_prep: the inputs of beta and of the decay are missing or too short");
  const int C = 2 * G * d + H * dv;
  GG_REQUIRE(x_stride >= C, "delta_prep: rows of %lld values hold no %d channels", x_stride, C);
  if (T == 0) return GG_OK;
  const int big = d > dv ? d : dv;
  GG_REQUIRE(big <= 8192, "delta_prep: head size %d is too large", big);
  const size_t smem = (size_t)(big + 33) * sizeof(float);
  const int threads = big >= 256 ? 256 : (big >= 128 ? 128 : 64);
  const dim3 grid(T, 2 * G + H + 1);
  GG_REQUIRE(grid.y <= 65535, "delta_prep: too many heads");
  if (dtype == GG_F32)
    gg_launch(delta_prep_kernel<float>, grid, dim3(threads), smem, stream, (const float*)x, x_stride, conv_w, (const float*)conv_state, zb, zb_stride, za, za_stride, dw, a_log, dt_bias, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, taps, qkv_out, beta, decay);
  else if (dtype == GG_BF16)
    gg_launch(delta_prep_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, (const __nv_bfloat16*)x, x_stride, conv_w, (const float*)conv_state, zb, zb_stride, za, za_stride, dw, a_log, dt_bias, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, taps, qkv_out, beta, decay);
  else
    return gg_fail(GG_ERR_INVALID, "delta_prep: unknown dtype %d", dtype);
  int rc = gg_check_launch("delta_prep");
  if (rc || taps == 1) return rc;
  return conv_state_update(x, x_stride, dtype, conv_state, cu_q_lens, context_lens, state_slots, B, C, taps, stream);
}

template <int DPT, bool CH, bool DELTA, int NC>
static int delta_recur_launch(const float* qkv, const float* beta, const float* decay, float* state,
                              const int* cu_q_lens, const int* context_lens, const int* state_slots, int B, int G, int H,
                              int d, int dv, float* o_raw, bool long_rows, cudaStream_t stream) {
  const int dp = DPT * DR_LANES;
  const size_t smem = (size_t)(2 * DR_STAGE_FLOATS_X(dp, CH, NC) + DR_CHUNK * DR_COLS * NC * DR_LANES) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_recur_kernel<DPT, CH, DELTA, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "delta_recur: %s", cudaGetErrorString(e));
  }
  const dim3 grid(B, H, (dv + DR_COLS * NC - 1) / (DR_COLS * NC));
  // A step with prompt portions: few blocks that run for as long as their sequence is, so they wait for an
  // empty machine (measured on a prompt of 2048 tokens with 128 blocks: 857 us launched early, 463 us so).
  if (long_rows)
    gg_launch_after(delta_recur_kernel<DPT, CH, DELTA, NC>, grid, dim3(DR_COLS * DR_LANES), smem, stream, qkv, beta, decay, state,
                    cu_q_lens, context_lens, state_slots, G, H, d, dv, o_raw);
  else
    gg_launch(delta_recur_kernel<DPT, CH, DELTA, NC>, grid, dim3(DR_COLS * DR_LANES), smem, stream, qkv, beta, decay, state, cu_q_lens,
              context_lens, state_slots, G, H, d, dv, o_raw);
  return gg_check_launch("delta_recur");
}

extern "C" int gg_delta_recur(const float* qkv, const float* beta, const float* decay, float* state,
                              const int* cu_q_lens, const int* context_lens, const int* state_slots, int B, int G, int H,
                              int d, int dv, int dw, int plain, int T, float* o_raw, cudaStream_t stream) {
  const bool long_rows = T > 4 * B;              // more than a few tokens a sequence: a step with prompt portions
  GG_REQUIRE(dw == 1 || dw == d, "delta_recur: a decay per head (1) or per key channel (%d), not %d", d, dw);
  GG_REQUIRE(!plain || dw == 1, "delta_recur: the plain recurrence takes a decay per head");
  GG_REQUIRE(B > 0 && G > 0 && H > 0 && H % G == 0 && d > 0 && dv > 0, "delta_recur: bad sizes B=%d G=%d H=%d d=%d dv=%d", B, G, H, d, dv);
  GG_REQUIRE(d <= 256, "delta_recur: key size %d is beyond 256", d);
  GG_REQUIRE(H <= 65535 && (dv + DR_COLS - 1) / DR_COLS <= 65535, "delta_recur: too many heads or columns");
#define DR_GO(N)                                                                                                              \
  do {                                                                                                                        \
    if (plain && N <= 16 && dv % (2 * DR_COLS) == 0)                                                                          \
      return delta_recur_launch<N, false, false, (N <= 16 ? 2 : 1)>(qkv, beta, decay, state, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, o_raw, long_rows, stream); \
    if (plain) return delta_recur_launch<N, false, false, 1>(qkv, beta, decay, state, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, o_raw, long_rows, stream); \
    if (dw > 1) return delta_recur_launch<N, true, true, 1>(qkv, beta, decay, state, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, o_raw, long_rows, stream); \
    return delta_recur_launch<N, false, true, 1>(qkv, beta, decay, state, cu_q_lens, context_lens, state_slots, B, G, H, d, dv, o_raw, long_rows, stream); \
  } while (0)
  if (d <= 16) DR_GO(2);
  if (d <= 32) DR_GO(4);
  if (d <= 64) DR_GO(8);
  if (d <= 128) DR_GO(16);
  DR_GO(32);
#undef DR_GO
}

extern "C" int gg_delta_out(const float* o_raw, const void* gate, long long gate_stride, int dtype, const float* w,
                            float eps, int T, int H, int dv, int gate_act, void* out, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && dv > 0 && H <= 65535, "delta_out: bad sizes T=%d H=%d dv=%d", T, H, dv);
  GG_REQUIRE(gate_act == 0 || gate_act == 1, "delta_out: the gate passes silu (0) or a sigmoid (1), not %d", gate_act);
  if (T == 0) return GG_OK;
  const int threads = dv >= 256 ? 256 : (dv >= 128 ? 128 : 64);
  const dim3 grid(T, H);
  if (dtype == GG_F32)
    gg_launch(delta_out_kernel<float>, grid, dim3(threads), 0, stream, o_raw, (const float*)gate, gate_stride, w, eps, H, dv, gate_act, (float*)out);
  else if (dtype == GG_BF16)
    gg_launch(delta_out_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, o_raw, (const __nv_bfloat16*)gate, gate_stride, w, eps, H, dv, gate_act, (__nv_bfloat16*)out);
  else
    return gg_fail(GG_ERR_INVALID, "delta_out: unknown dtype %d", dtype);
  return gg_check_launch("delta_out");
}
