// Routing of a mixture of experts, on the device from start to end (a step never asks the host
// how many tokens an expert got, so a step of decoded tokens can be captured and replayed).
//
// gg_moe_route:   z[t, e] = h[t] . Wr[e] + b[e] in float32; the `top` largest logits of a token
//                 (ties: the lower index) are its experts, weights = softmax over those alone, or
//                 the softmax over all experts renormalised over the chosen; optionally only
//                 experts of the best groups can be chosen (moe_pick)
// gg_moe_align:   the (token, choice) pairs sorted by expert: offsets[e] .. offsets[e+1] are the
//                 places of expert e in `sorted` (values t * top + j), `place` is the inverse
// gg_moe_combine: out[t] = sum_j weight[t, j] * y[place[t * top + j]] (+ shared[t]), float32 sums
//                 in the order of j
// The products between them are gg_grouped_gemm's (grouped_gemm.cu).
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 32

// A block routes ROUTE_TOK tokens: their rows are staged in shared memory as float32, and a warp
// that takes an expert reads that expert's router row once (16 bytes a lane at a time) for all of
// them, so the router's weights cross from L2 once per ROUTE_TOK tokens and not once per token.
#define ROUTE_TOK 4      // for steps of many tokens; steps of a few tokens take one token a block, for more blocks

__device__ __forceinline__ void route_load(const float* w, float (&v)[8], int n) {
  const float4 a = *reinterpret_cast<const float4*>(w);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  (void)n;
}
__device__ __forceinline__ void route_load(const __nv_bfloat16* w, float (&v)[8], int n) {
  const uint4 r = *reinterpret_cast<const uint4*>(w);
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 b = __bfloat1622float2(p[j]); v[2 * j] = b.x; v[2 * j + 1] = b.y; }
  (void)n;
}

// One warp picks a token's experts from its logits zr[E] (shared memory, overwritten) and weighs them.
// weigh = 0: weights = softmax over the chosen logits alone.  weigh = 1: scores = softmax over all
// experts, weights = the chosen scores divided by their sum (+ 1e-20).  groups > 1: the experts form
// that many equal groups of neighbours, a group's score is its best expert's, and only experts of the
// `keep` best groups can be chosen.  Ties: the lower index.
__device__ __forceinline__ void moe_pick(float* zr, int E, int top, int weigh, int groups, int keep, int lane,
                                         int* __restrict__ idx, float* __restrict__ wgt) {
  float zmax = 0.f, zsum = 1.f;
  if (weigh == 1) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sm = 0.f;
    for (int e = lane; e < E; e += 32) sm += expf(zr[e] - m);
    zmax = m; zsum = warp_sum(sm);
  }
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    unsigned kept = 0;                             // bit i: group lane + 32 i is kept
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int bg = 0x7fffffff;
      for (int g = lane, i = 0; g < groups; g += 32, ++i) {
        if (kept >> i & 1u) continue;
        float gm = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) gm = fmaxf(gm, zr[e]);
        if (gm > best || (gm == best && g < bg)) { best = gm; bg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (ov > best || (ov == best && og < bg)) { best = ov; bg = og; }
      }
      if (bg == 0x7fffffff) break;                 // nothing but NaN left
      if ((bg & 31) == lane) kept |= 1u << (bg >> 5);
    }
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane, g = e < E ? e / per : 0;
      const unsigned owner = __shfl_sync(0xffffffffu, kept, g & 31);
      if (e < E && !(owner >> (g >> 5) & 1u)) zr[e] = -INFINITY;
    }
    __syncwarp();
  }
  float val[MOE_MAX_TOP];
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = zr[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;                    // every logit left is -inf or NaN
    val[j] = best;
    if (lane == 0) { idx[j] = bi; zr[bi] = -INFINITY; }
    __syncwarp();
  }
  if (lane == 0) {
    if (weigh == 1) {
      float sum = 0.f;
      for (int j = 0; j < top; ++j) { val[j] = expf(val[j] - zmax) / zsum; sum += val[j]; }
      for (int j = 0; j < top; ++j) wgt[j] = val[j] / (sum + 1e-20f);
    } else {
      const float m = val[0];                        // the largest comes first
      float sum = 0.f;
      for (int j = 0; j < top; ++j) { val[j] = expf(val[j] - m); sum += val[j]; }
      for (int j = 0; j < top; ++j) wgt[j] = val[j] / sum;
    }
  }
}

template <typename TA, int TOK>
__global__ void moe_route_kernel(const TA* __restrict__ h, const TA* __restrict__ wr, const float* __restrict__ bias,
                                 int T, int D, int E, int top, int weigh, int groups, int keep,
                                 int* __restrict__ idx, float* __restrict__ wgt, int vec) {
  __shared__ float z[TOK][MOE_MAX_EXPERTS];
  extern __shared__ __align__(16) float xs[];              // TOK rows of D floats
  constexpr int VPT = 16 / (int)sizeof(TA);
  pdl_trigger();
  pdl_wait();
  const int t0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int nt = min(TOK, T - t0);
  for (int e = threadIdx.x; e < TOK * D; e += blockDim.x) {
    const int r = e / D;
    xs[e] = r < nt ? to_f32(h[(size_t)(t0 + r) * D + (e - r * D)]) : 0.f;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const TA* w = wr + (size_t)e * D;
    float s[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) s[r] = 0.f;
    if (vec) {
      for (int c = lane * VPT; c < D; c += 32 * VPT) {
        float v[8];
        route_load(w + c, v, VPT);
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
#pragma unroll
          for (int j = 0; j < VPT; j += 4) {                // the staged rows four values at a time
            const float4 x = *reinterpret_cast<const float4*>(xs + r * D + c + j);
            s[r] = fmaf(x.x, v[j], s[r]); s[r] = fmaf(x.y, v[j + 1], s[r]);
            s[r] = fmaf(x.z, v[j + 2], s[r]); s[r] = fmaf(x.w, v[j + 3], s[r]);
          }
        }
      }
    } else {
      for (int c = lane; c < D; c += 32) {
        const float v = to_f32(w[c]);
#pragma unroll
        for (int r = 0; r < TOK; ++r) s[r] = fmaf(xs[r * D + c], v, s[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      const float tot = warp_sum(s[r]);
      if (lane == 0) z[r][e] = tot + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (warp < nt)                                           // warp r picks for token t0 + r (the block has TOK warps or more)
    moe_pick(z[warp], E, top, weigh, groups, keep, lane, idx + (size_t)(t0 + warp) * top, wgt + (size_t)(t0 + warp) * top);
}

// The choice alone, from logits a product has already made (long steps: z = h Wr^T in float32 by the
// vendor library from the bfloat16 rows): one warp a token adds the bias, picks and weighs.
__global__ void moe_topk_kernel(const float* __restrict__ z, const float* __restrict__ bias, int T, int E, int top,
                                int weigh, int groups, int keep, int* __restrict__ idx, float* __restrict__ wgt) {
  extern __shared__ float zs[];                            // warps x E
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* zr = zs + warp * E;
  for (int e = lane; e < E; e += 32) zr[e] = z[(size_t)t * E + e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  moe_pick(zr, E, top, weigh, groups, keep, lane, idx + (size_t)t * top, wgt + (size_t)t * top);
}

// One CTA.  counts and cursors in shared memory; the order of the rows inside an expert's range
// is whatever the atomics give, which no result depends on.  pad > 1: every expert's range
// starts at a multiple of pad (the places between its last row and the next range hold -1 in
// `sorted`), `slots` is the length of `sorted`, and tile_group[i] is the expert that places
// pad * i .. pad * i + pad - 1 belong to, or -1 past the last range (n_tiles entries).
__global__ void moe_align_kernel(const int* __restrict__ idx, int n, int E, int pad, int slots, int* __restrict__ offsets,
                                 int* __restrict__ sorted, int* __restrict__ place, int* __restrict__ tile_group,
                                 int n_tiles) {
  __shared__ int cnt[MOE_MAX_EXPERTS + 1];
  __shared__ int start[MOE_MAX_EXPERTS + 1];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  if (pad > 1)
    for (int i = threadIdx.x; i < slots; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      cnt[e] = run; start[e] = run; offsets[e] = run;
      run += (c + pad - 1) / pad * pad;
    }
    start[E] = run; offsets[E] = run;
  }
  __syncthreads();
  if (tile_group)
    for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
      const int p = i * pad;
      int g = -1;
      if (p < start[E]) {
        int lo = 0, hi = E;                          // the last expert whose range starts at or before p
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (start[mid] <= p) lo = mid; else hi = mid; }
        g = lo;
      }
      tile_group[i] = g;
    }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cnt[idx[i]], 1);
    sorted[p] = i;
    place[i] = p;
  }
}

// xs[p] = x[sorted[p] / top] for the places that hold a pair, zeros for the others: the rows of
// every expert gathered into one block that starts at a multiple of the product's tile height.
template <typename TA>
__global__ void moe_gather_kernel(const TA* __restrict__ x, const int* __restrict__ sorted, int top, int D,
                                  TA* __restrict__ xs, int vec) {
  pdl_trigger();
  pdl_wait();
  const size_t p = blockIdx.x;
  const int src = sorted[p];
  TA* o = xs + p * D;
  if (vec) {
    constexpr int VPT = 16 / (int)sizeof(TA);
    const uint4* in = src >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)(src / top) * D) : nullptr;
    for (int c = threadIdx.x; c < D / VPT; c += blockDim.x)
      reinterpret_cast<uint4*>(o)[c] = in ? in[c] : make_uint4(0, 0, 0, 0);
  } else {
    const TA* in = src >= 0 ? x + (size_t)(src / top) * D : nullptr;
    for (int c = threadIdx.x; c < D; c += blockDim.x) o[c] = in ? in[c] : from_f32<TA>(0.f);
  }
}

template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wgt,
                                   const TA* __restrict__ shared_out, TA* __restrict__ out, int D, int top) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  if (D % 4 == 0) {                              // rows of every buffer are then 8-byte aligned at least
    for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      for (int j = 0; j < top; ++j) {
        const float w = wgt[t * top + j];
        const TA* r = y + (size_t)place[t * top + j] * D + c;
        s0 = fmaf(w, to_f32(r[0]), s0); s1 = fmaf(w, to_f32(r[1]), s1);
        s2 = fmaf(w, to_f32(r[2]), s2); s3 = fmaf(w, to_f32(r[3]), s3);
      }
      if (shared_out) {
        const TA* r = shared_out + t * D + c;
        s0 += to_f32(r[0]); s1 += to_f32(r[1]); s2 += to_f32(r[2]); s3 += to_f32(r[3]);
      }
      TA* o = out + t * D + c;
      o[0] = from_f32<TA>(s0); o[1] = from_f32<TA>(s1); o[2] = from_f32<TA>(s2); o[3] = from_f32<TA>(s3);
    }
    return;
  }
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < top; ++j)
      s = fmaf(wgt[t * top + j], to_f32(y[(size_t)place[t * top + j] * D + c]), s);
    if (shared_out) s += to_f32(shared_out[t * D + c]);
    out[t * D + c] = from_f32<TA>(s);
  }
}

static int check_pick(const char* who, int E, int top, int weigh, int groups, int keep) {
  GG_REQUIRE(weigh == 0 || weigh == 1, "%s: unknown way %d of weighing the chosen experts", who, weigh);
  GG_REQUIRE(groups >= 1 && keep >= 1 && keep <= groups && E % groups == 0, "%s: %d experts in %d groups of which %d are kept", who, E, groups, keep);
  GG_REQUIRE(top <= keep * (E / groups), "%s: %d choices from %d groups of %d experts", who, top, keep, E / groups);
  return GG_OK;
}

extern "C" int gg_moe_route(const void* h, const void* wr, const float* bias, int T, int D, int E, int top,
                            int weigh, int groups, int keep, int* idx, float* wgt, int act_dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && D > 0 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes T=%d D=%d E=%d top=%d", T, D, E, top);
  GG_REQUIRE(E <= MOE_MAX_EXPERTS && top <= MOE_MAX_TOP, "moe_route: at most %d experts and %d choices a token (got %d, %d)",
             MOE_MAX_EXPERTS, MOE_MAX_TOP, E, top);
  GG_REQUIRE(h && wr && idx && wgt, "moe_route: a pointer is null");
  if (int rc = check_pick("moe_route", E, top, weigh, groups, keep)) return rc;
  if (T == 0) return GG_OK;
  const int tok = T > 256 ? ROUTE_TOK : 1;
  const size_t smem = (size_t)tok * D * sizeof(float);
  GG_REQUIRE(smem <= 200 * 1024, "moe_route: rows of %d values do not fit in shared memory", D);
  const int vec = (act_dtype == GG_F32 ? D % 4 == 0 : D % 8 == 0) && ((size_t)wr % 16) == 0;
  const int threads = E >= 8 ? 256 : 128;                  // at least ROUTE_TOK warps
  const int blocks = (T + tok - 1) / tok;
#define ROUTE_LAUNCH(T_, N_)                                                                                     \
  do {                                                                                                           \
    if (smem > 28 * 1024) cudaFuncSetAttribute(moe_route_kernel<T_, N_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    gg_launch(moe_route_kernel<T_, N_>, dim3(blocks), dim3(threads), smem, stream, (const T_*)h, (const T_*)wr, bias, T, D, E, top, weigh, groups, keep, idx, wgt, vec); \
  } while (0)
  if (act_dtype == GG_F32) {
    if (tok == 1) ROUTE_LAUNCH(float, 1); else ROUTE_LAUNCH(float, ROUTE_TOK);
  } else if (act_dtype == GG_BF16) {
    if (tok == 1) ROUTE_LAUNCH(__nv_bfloat16, 1); else ROUTE_LAUNCH(__nv_bfloat16, ROUTE_TOK);
  } else
    return gg_fail(GG_ERR_INVALID, "moe_route: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_route");
}

extern "C" int gg_moe_topk(const float* z, const float* bias, int T, int E, int top, int weigh, int groups, int keep,
                           int* idx, float* wgt, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && E > 0 && top > 0 && top <= E && E <= MOE_MAX_EXPERTS && top <= MOE_MAX_TOP,
             "moe_topk: bad sizes T=%d E=%d top=%d", T, E, top);
  GG_REQUIRE(z && idx && wgt, "moe_topk: a pointer is null");
  if (int rc = check_pick("moe_topk", E, top, weigh, groups, keep)) return rc;
  if (T == 0) return GG_OK;
  const int warps = 4;
  gg_launch(moe_topk_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), (size_t)warps * E * sizeof(float), stream,
            z, bias, T, E, top, weigh, groups, keep, idx, wgt);
  return gg_check_launch("moe_topk");
}

extern "C" int gg_moe_align(const int* idx, int n, int E, int pad, int slots, int* offsets, int* sorted, int* place,
                            int* tile_group, int n_tiles, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && E > 0 && E <= MOE_MAX_EXPERTS && pad >= 1, "moe_align: bad sizes n=%d E=%d pad=%d", n, E, pad);
  GG_REQUIRE(idx && offsets && sorted && place, "moe_align: a pointer is null");
  GG_REQUIRE(pad == 1 || (long long)slots >= (long long)n + (long long)E * (pad - 1),
             "moe_align: %d places do not hold %d rows of %d experts padded to %d", slots, n, E, pad);
  GG_REQUIRE(!tile_group || (long long)n_tiles * pad >= slots, "moe_align: %d tile entries for %d places", n_tiles, slots);
  gg_launch(moe_align_kernel, dim3(1), dim3(1024), 0, stream, idx, n, E, pad, slots, offsets, sorted, place, tile_group, n_tiles);
  return gg_check_launch("moe_align");
}

extern "C" int gg_moe_gather(const void* x, const int* sorted, int slots, int top, int D, void* xs, int act_dtype,
                             cudaStream_t stream) {
  GG_REQUIRE(slots >= 0 && top > 0 && D > 0 && x && sorted && xs, "moe_gather: bad arguments");
  if (slots == 0) return GG_OK;
  const int vpt = act_dtype == GG_F32 ? 4 : 8;
  const int vec = D % vpt == 0 && ((size_t)x % 16) == 0 && ((size_t)xs % 16) == 0;
  if (act_dtype == GG_F32)
    gg_launch(moe_gather_kernel<float>, dim3(slots), dim3(128), 0, stream, (const float*)x, sorted, top, D, (float*)xs, vec);
  else if (act_dtype == GG_BF16)
    gg_launch(moe_gather_kernel<__nv_bfloat16>, dim3(slots), dim3(128), 0, stream, (const __nv_bfloat16*)x, sorted, top, D,
              (__nv_bfloat16*)xs, vec);
  else
    return gg_fail(GG_ERR_INVALID, "moe_gather: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_gather");
}

extern "C" int gg_moe_combine(const void* y, const int* place, const float* wgt, const void* shared_out, void* out,
                              int T, int D, int top, int act_dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && D > 0 && top > 0, "moe_combine: bad sizes T=%d D=%d top=%d", T, D, top);
  GG_REQUIRE(y && place && wgt && out, "moe_combine: a pointer is null");
  if (T == 0) return GG_OK;
  const int threads = D >= 1024 ? 256 : 128;
  if (act_dtype == GG_F32)
    gg_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)y, place, wgt, (const float*)shared_out,
              (float*)out, D, top);
  else if (act_dtype == GG_BF16)
    gg_launch(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)y, place, wgt,
              (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out, D, top);
  else
    return gg_fail(GG_ERR_INVALID, "moe_combine: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_combine");
}
