// Norms with a mean and a bias, and the norm that sits on a sublayer's OUTPUT.
//
//   layer norm:  n(x) = (x - mean(x)) / sqrt(mean((x - mean)^2) + eps) * w + b
//   rms norm:    n(x) = x / sqrt(mean(x^2) + eps) * w                     (layer = 0, b = null)
//
// gg_add_norm:        x = resid[r] (+ delta[r]); out[i] = TA(n(x))        (the norm ahead of a product
//                     or of the head; r = rows ? rows[i] : i)
// gg_norm_scale_add:  resid[t] += scale * n(y[t]);  copy[t] = TA(resid[t])
//                     (a block that norms what a sublayer returns, scales it per channel and adds it
//                     to the residual stream; the next sublayer reads the stream itself, so its
//                     rounding to the activation type is made here too)
//
// Statistics, the affine part, the scaling and the residual sum are float32; the variance is
// taken about the mean in a second pass over the row held in shared memory.
#include "common.cuh"

// four values at a time (rows of a multiple of four values, 16-byte aligned in float32)
template <typename TA> struct LnVec4;
template <> struct LnVec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct LnVec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&a);
    r.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename TA>
__global__ void add_norm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                const float* __restrict__ w, const float* __restrict__ b,
                                TA* __restrict__ out, const int* __restrict__ rows, int H, float eps,
                                int write_back, int layer) {
  extern __shared__ __align__(16) float xs[];          // H floats + 33 for the reduction
  float* red = xs + H;
  pdl_trigger();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  pdl_wait();
  float* xr = resid + (size_t)r * H;
  const TA* dr = delta ? delta + (size_t)r * H : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float x = xr[c];
    if (dr) {
      x += to_f32(dr[c]);
      if (write_back) xr[c] = x;
    }
    xs[c] = x;
    s += x;
  }
  const float mean = layer ? block_sum(s, red) / (float)H : 0.f;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float dx = xs[c] - mean;
    ss += dx * dx;
  }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  TA* o = out + (size_t)i * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float n = (xs[c] - mean) * rinv * w[c];
    if (b) n += b[c];
    o[c] = from_f32<TA>(n);
  }
}

template <typename TA, bool VEC>
__global__ void norm_scale_add_kernel(float* __restrict__ resid, const TA* __restrict__ y,
                                      const float* __restrict__ w, const float* __restrict__ b,
                                      const float* __restrict__ scale, TA* __restrict__ copy, int H,
                                      float eps, int layer) {
  extern __shared__ __align__(16) float xs[];
  float* red = xs + H;
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const TA* yr = y + t * H;
  float s = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      const float4 x = LnVec4<TA>::load(yr + c);
      *reinterpret_cast<float4*>(xs + c) = x;
      s += (x.x + x.y) + (x.z + x.w);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float x = to_f32(yr[c]);
      xs[c] = x;
      s += x;
    }
  }
  const float mean = layer ? block_sum(s, red) / (float)H : 0.f;
  float ss = 0.f;
  if (!layer) __syncthreads();                 // block_sum was the barrier between writing xs and reading it
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float dx = xs[c] - mean;
    ss += dx * dx;
  }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  float* xr = resid + t * H;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      const float4 x = *reinterpret_cast<const float4*>(xs + c), g = *reinterpret_cast<const float4*>(w + c);
      float4 n = make_float4((x.x - mean) * rinv * g.x, (x.y - mean) * rinv * g.y, (x.z - mean) * rinv * g.z, (x.w - mean) * rinv * g.w);
      if (b) { const float4 q = *reinterpret_cast<const float4*>(b + c); n.x += q.x; n.y += q.y; n.z += q.z; n.w += q.w; }
      if (scale) { const float4 q = *reinterpret_cast<const float4*>(scale + c); n.x *= q.x; n.y *= q.y; n.z *= q.z; n.w *= q.w; }
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      v.x += n.x; v.y += n.y; v.z += n.z; v.w += n.w;
      *reinterpret_cast<float4*>(xr + c) = v;
      if (copy) LnVec4<TA>::store(copy + t * H + c, v);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float n = (xs[c] - mean) * rinv * w[c];
      if (b) n += b[c];
      if (scale) n *= scale[c];
      const float v = xr[c] + n;
      xr[c] = v;
      if (copy) copy[t * H + c] = from_f32<TA>(v);
    }
  }
}

// copy[t] = TA(resid[t]): the rows a sublayer reads when it takes the residual stream itself.
template <typename TA>
__global__ void cast_rows_kernel(const float* __restrict__ resid, TA* __restrict__ copy, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x)
    copy[e] = from_f32<TA>(resid[e]);
}

static int norm_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

template <typename K> static int norm_smem(K kernel, size_t smem, const char* who) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
  }
  return GG_OK;
}

extern "C" int gg_add_norm(float* resid, const void* delta, const float* w, const float* b, void* out,
                           int act_dtype, const int* rows, int n, int H, float eps, int write_back,
                           int layer, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && H > 0 && eps >= 0.f, "add_norm: bad sizes n=%d H=%d eps=%g", n, H, (double)eps);
  GG_REQUIRE(resid && w && out, "add_norm: residual, weight and output are needed");
  if (n == 0) return GG_OK;
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  GG_REQUIRE(smem <= 227 * 1024, "add_norm: width %d needs %zu B of shared memory", H, smem);
  int rc;
  if (act_dtype == GG_F32) {
    if ((rc = norm_smem(add_norm_kernel<float>, smem, "add_norm"))) return rc;
    gg_launch(add_norm_kernel<float>, dim3(n), dim3(norm_threads(H)), smem, stream, resid, (const float*)delta, w, b,
              (float*)out, rows, H, eps, write_back, layer);
  } else if (act_dtype == GG_BF16) {
    if ((rc = norm_smem(add_norm_kernel<__nv_bfloat16>, smem, "add_norm"))) return rc;
    gg_launch(add_norm_kernel<__nv_bfloat16>, dim3(n), dim3(norm_threads(H)), smem, stream, resid,
              (const __nv_bfloat16*)delta, w, b, (__nv_bfloat16*)out, rows, H, eps, write_back, layer);
  } else {
    return gg_fail(GG_ERR_INVALID, "add_norm: unknown dtype %d", act_dtype);
  }
  return gg_check_launch("add_norm");
}

extern "C" int gg_norm_scale_add(float* resid, const void* y, const float* w, const float* b,
                                 const float* scale, void* copy, int act_dtype, int T, int H, float eps,
                                 int layer, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && eps >= 0.f, "norm_scale_add: bad sizes T=%d H=%d eps=%g", T, H, (double)eps);
  GG_REQUIRE(resid && y && w, "norm_scale_add: residual, input and weight are needed");
  if (T == 0) return GG_OK;
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  GG_REQUIRE(smem <= 227 * 1024, "norm_scale_add: width %d needs %zu B of shared memory", H, smem);
  int rc;
  const size_t esz = act_dtype == GG_F32 ? 4 : 2;
  const bool vec = H % 4 == 0 && ((size_t)resid % 16) == 0 && ((size_t)w % 16) == 0 && ((size_t)b % 16) == 0 &&
                   ((size_t)scale % 16) == 0 && ((size_t)y % (4 * esz)) == 0 && ((size_t)copy % (4 * esz)) == 0;
  const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : norm_threads(H);
#define NSA_LAUNCH(T_, V_)                                                                                    \
  do {                                                                                                        \
    if ((rc = norm_smem(norm_scale_add_kernel<T_, V_>, smem, "norm_scale_add"))) return rc;                   \
    gg_launch(norm_scale_add_kernel<T_, V_>, dim3(T), dim3(threads), smem, stream, resid, (const T_*)y, w, b, \
              scale, (T_*)copy, H, eps, layer);                                                               \
  } while (0)
  if (act_dtype == GG_F32) {
    if (vec) NSA_LAUNCH(float, true); else NSA_LAUNCH(float, false);
  } else if (act_dtype == GG_BF16) {
    if (vec) NSA_LAUNCH(__nv_bfloat16, true); else NSA_LAUNCH(__nv_bfloat16, false);
  } else {
    return gg_fail(GG_ERR_INVALID, "norm_scale_add: unknown dtype %d", act_dtype);
  }
  return gg_check_launch("norm_scale_add");
}

extern "C" int gg_cast_rows(const float* resid, void* copy, int act_dtype, long long n, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && resid && copy, "cast_rows: bad arguments");
  if (n == 0) return GG_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act_dtype == GG_F32)
    gg_launch(cast_rows_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, resid, (float*)copy, (size_t)n);
  else if (act_dtype == GG_BF16)
    gg_launch(cast_rows_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, resid, (__nv_bfloat16*)copy, (size_t)n);
  else
    return gg_fail(GG_ERR_INVALID, "cast_rows: unknown dtype %d", act_dtype);
  return gg_check_launch("cast_rows");
}


// resid[t] += n(x[t]) with x = (y[t] + yb) * sigmoid(g[t] + gb), n the RMS norm with weight w: a block whose
// sublayers' results pass a learned gate (g = a product of the sublayer's own input, gb its bias) and then a
// norm before they join the residual stream.  yb: a bias of the sublayer's last product that was left to this
// kernel (null: none); g null: no gate.  The gate, the statistics and the sum are float32.
template <typename TA>
__global__ void gate_norm_add_kernel(float* __restrict__ resid, const TA* __restrict__ y, const float* __restrict__ yb,
                                     const TA* __restrict__ g, long long g_stride, const float* __restrict__ gb,
                                     const float* __restrict__ w, int H, float eps) {
  extern __shared__ __align__(16) float xs[];
  float* red = xs + H;
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float x = to_f32(y[t * H + c]) + (yb ? yb[c] : 0.f);
    if (g) x /= 1.f + expf(-(to_f32(g[t * g_stride + c]) + (gb ? gb[c] : 0.f)));
    xs[c] = x;
    ss += x * x;
  }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  float* xr = resid + t * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) xr[c] += xs[c] * rinv * w[c];
}

// The same with the row in registers: four neighbouring values at a time, up to GNA_VECS such groups a thread
// (one round of loads, one block sum, one round over the residual: what a step of few tokens is bound by).
#define GNA_VECS 4
template <typename TA>
__global__ void __launch_bounds__(1024)
gate_norm_add_vec_kernel(float* __restrict__ resid, const TA* __restrict__ y, const float* __restrict__ yb,
                         const TA* __restrict__ g, long long g_stride, const float* __restrict__ gb,
                         const float* __restrict__ w, int H, float eps) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  float4 x[GNA_VECS];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < GNA_VECS; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 4;
    x[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < H) {
      float4 v = LnVec4<TA>::load(y + t * H + c);
      if (yb) { const float4 b = *reinterpret_cast<const float4*>(yb + c); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
      if (g) {
        float4 z = LnVec4<TA>::load(g + t * g_stride + c);
        if (gb) { const float4 b = *reinterpret_cast<const float4*>(gb + c); z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w; }
        v.x /= 1.f + expf(-z.x); v.y /= 1.f + expf(-z.y); v.z /= 1.f + expf(-z.z); v.w /= 1.f + expf(-z.w);
      }
      x[k] = v;
      ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
  }
  const float rinv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  float* xr = resid + t * H;
#pragma unroll
  for (int k = 0; k < GNA_VECS; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 4;
    if (c < H) {
      const float4 q = *reinterpret_cast<const float4*>(w + c);
      float4 r = *reinterpret_cast<const float4*>(xr + c);
      r.x += x[k].x * rinv * q.x; r.y += x[k].y * rinv * q.y; r.z += x[k].z * rinv * q.z; r.w += x[k].w * rinv * q.w;
      *reinterpret_cast<float4*>(xr + c) = r;
    }
  }
}

extern "C" int gg_gate_norm_add(float* resid, const void* y, const float* yb, const void* g, long long g_stride,
                                const float* gb, const float* w, int act_dtype, int T, int H, float eps, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && H > 0 && eps >= 0.f, "gate_norm_add: bad sizes T=%d H=%d eps=%g", T, H, (double)eps);
  GG_REQUIRE(resid && y && w && (!g || g_stride >= H), "gate_norm_add: residual, input and weight are needed");
  if (T == 0) return GG_OK;
  const size_t esize = act_dtype == GG_F32 ? 4 : 2;
  if ((act_dtype == GG_F32 || act_dtype == GG_BF16) && H % 4 == 0 && H <= 4 * GNA_VECS * 1024 && (g_stride * esize) % (4 * esize) == 0 &&
      ((size_t)y % 16) == 0 && ((size_t)g % (4 * esize)) == 0 && ((size_t)resid % 16) == 0 && ((size_t)w % 16) == 0 &&
      ((size_t)yb % 16) == 0 && ((size_t)gb % 16) == 0) {
    int threads = ((H / 4 + GNA_VECS - 1) / GNA_VECS + 31) / 32 * 32;        // as few rounds a thread as the row allows
    if (H / 4 <= 1024) threads = (H / 4 + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (act_dtype == GG_F32)
      gg_launch(gate_norm_add_vec_kernel<float>, dim3(T), dim3(threads), 0, stream, resid, (const float*)y, yb, (const float*)g, g_stride, gb, w, H, eps);
    else
      gg_launch(gate_norm_add_vec_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, resid, (const __nv_bfloat16*)y, yb, (const __nv_bfloat16*)g, g_stride, gb, w, H, eps);
    return gg_check_launch("gate_norm_add");
  }
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  GG_REQUIRE(smem <= 200 * 1024, "gate_norm_add: rows of %d values do not fit in shared memory", H);
  const int threads = H >= 2048 ? 512 : 256;
  if (act_dtype == GG_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(gate_norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gg_launch(gate_norm_add_kernel<float>, dim3(T), dim3(threads), smem, stream, resid, (const float*)y, yb, (const float*)g, g_stride, gb, w, H, eps);
  } else if (act_dtype == GG_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(gate_norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gg_launch(gate_norm_add_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, resid, (const __nv_bfloat16*)y, yb, (const __nv_bfloat16*)g, g_stride, gb, w, H, eps);
  } else {
    return gg_fail(GG_ERR_INVALID, "gate_norm_add: unknown dtype %d", act_dtype);
  }
  return gg_check_launch("gate_norm_add");
}
