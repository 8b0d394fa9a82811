// Memory-bound row kernels: embedding gather, RMSNorm (plain, gathered, and added to the
// residual), SwiGLU, residual add, row gather.  The residual stream is always float; the
// template parameter is the type of the activations that feed the matrix products.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_err[512];

int leb_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return 1;
}
LEB_API const char* leb_last_error() { return g_err; }

long long g_leb_launches = 0;
int g_leb_pdl = 1;
thread_local int g_leb_gate_act = 0;
LEB_API void leb_set_pdl(int on) { g_leb_pdl = on ? 1 : 0; }
LEB_API long long leb_launch_count() { return g_leb_launches; }

// ---------------------------------------------------------------------------------------------
// x[m, :] = table[tokens[m], :]            (reference: src/dense.rs:172-177 takes the row as is)
template <typename T>
__global__ void embed_kernel(float* __restrict__ x, const T* __restrict__ table,
                             const int* __restrict__ tokens, int D, int V, float scale) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int m = blockIdx.x;
  int tok = tokens[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);  // ids are validated on the host; never read outside
  const T* row = table + (size_t)tok * D;
  float* o = x + (size_t)m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = to_f32(row[i]) * scale;   // scale 1 leaves the row as it is
}

LEB_API int leb_embed(float* x, const void* table, int table_dtype, const int* tokens, int M, int D,
                      int V, float scale, cudaStream_t st) {
  if (M <= 0) return 0;
  int threads = D >= 1024 ? 256 : 128;
  if (table_dtype == LEB_F32)
    leb_launch(embed_kernel<float>, dim3(M), dim3(threads), 0, st, x, (const float*)table, tokens, D, V, scale);
  else if (table_dtype == LEB_BF16)
    leb_launch(embed_kernel<bf16>, dim3(M), dim3(threads), 0, st, x, (const bf16*)table, tokens, D, V, scale);
  else
    return leb_fail("leb_embed: unknown table dtype %d", table_dtype);
  LEB_CHECK_LAUNCH("leb_embed");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm:  r = rsqrt(mean(x^2) + eps);  y = x * r * w      (src/dense.rs:27-30: eps inside the
// root, added to the mean; the weight multiplies directly).  Sum, root and product are float.
//   rows != null : input row m is x[rows[m]]  (the rows whose logits are wanted)
//   ADD          : out (float) += y           (a norm after the mixer or feed-forward, src/dense.rs:185,192)
template <typename TO, bool ADD>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows, int D,
                               float eps) {
  __shared__ float red[33];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int m = blockIdx.x;
  const float* xi = x + (size_t)(rows ? rows[m] : m) * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = xi[i];
    s += v * v;
  }
  s = block_sum(s, red);
  float r = 1.0f / sqrtf(s / (float)D + eps);
  TO* o = out + (size_t)m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float y = xi[i] * r * w[i];
    if (ADD)
      o[i] = from_f32<TO>(to_f32(o[i]) + y);
    else
      o[i] = from_f32<TO>(y);
  }
}

// The same norm for bfloat16 output with 16-byte loads: a thread keeps its CH float4 pieces of
// the row in registers between the sum and the product, so the row is read once.
template <int CH>
__global__ void __launch_bounds__(256)
rmsnorm_bf16_vec_kernel(bf16* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                        const int* __restrict__ rows, int D, float eps) {
  __shared__ float red[33];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m = blockIdx.x;
  const float4* xi = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[m] : m) * D);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const int n4 = D >> 2;
  float4 v[CH];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * 256;
    if (i < n4) {
      v[c] = xi[i];
      s += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
    }
  }
  s = block_sum(s, red);
  const float r = 1.0f / sqrtf(s / (float)D + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)m * D);
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * 256;
    if (i < n4) {
      const float4 ww = w4[i];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[c].x * r * ww.x, v[c].y * r * ww.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[c].z * r * ww.z, v[c].w * r * ww.w);
      o[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

LEB_API int leb_rmsnorm(void* out, int out_dtype, const float* x, const float* w, const int* rows,
                        int M, int D, float eps, int add, cudaStream_t st) {
  if (M <= 0) return 0;
  if (!add && out_dtype == LEB_BF16 && D % 4 == 0 && D <= 8192 && ((uintptr_t)x % 16) == 0 &&
      ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 8) == 0) {
    const int ch = ceil_div(D / 4, 256);
    bf16* o = (bf16*)out;
    if (ch <= 1) leb_launch(rmsnorm_bf16_vec_kernel<1>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else if (ch <= 2) leb_launch(rmsnorm_bf16_vec_kernel<2>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else if (ch <= 4) leb_launch(rmsnorm_bf16_vec_kernel<4>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else leb_launch(rmsnorm_bf16_vec_kernel<8>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    LEB_CHECK_LAUNCH("leb_rmsnorm");
    return 0;
  }
  int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  if (add) {
    LEB_REQUIRE(out_dtype == LEB_F32, "leb_rmsnorm: the added form writes the float residual");
    leb_launch(rmsnorm_kernel<float, true>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, rows, D, eps);
  } else if (out_dtype == LEB_F32) {
    leb_launch(rmsnorm_kernel<float, false>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, rows, D, eps);
  } else if (out_dtype == LEB_BF16) {
    leb_launch(rmsnorm_kernel<bf16, false>, dim3(M), dim3(threads), 0, st, (bf16*)out, x, w, rows, D, eps);
  } else {
    return leb_fail("leb_rmsnorm: unknown output dtype %d", out_dtype);
  }
  LEB_CHECK_LAUNCH("leb_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// a[m, j] = silu(gu[m, j]) * gu[m, F + j],  silu(x) = x / (1 + exp(-x))   (src/dense.rs:31,190)
template <typename TI, typename TO>
__global__ void swiglu_kernel(TO* __restrict__ a, const TI* __restrict__ gu, int F, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t m = i / F;
  int j = (int)(i - m * F);
  float g = to_f32(gu[m * 2 * F + j]);
  float u = to_f32(gu[m * 2 * F + F + j]);
  a[i] = from_f32<TO>(silu_mul<TO>(g, u));
}

LEB_API int leb_swiglu(void* a, int out_dtype, const void* gu, int in_dtype, int M, int F,
                       cudaStream_t st) {
  size_t total = (size_t)M * F;
  if (total == 0) return 0;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (in_dtype == LEB_F32 && out_dtype == LEB_F32)
    swiglu_kernel<float, float><<<blocks, 256, 0, st>>>((float*)a, (const float*)gu, F, total);
  else if (in_dtype == LEB_F32 && out_dtype == LEB_BF16)
    swiglu_kernel<float, bf16><<<blocks, 256, 0, st>>>((bf16*)a, (const float*)gu, F, total);
  else if (in_dtype == LEB_BF16 && out_dtype == LEB_BF16)
    swiglu_kernel<bf16, bf16><<<blocks, 256, 0, st>>>((bf16*)a, (const bf16*)gu, F, total);
  else
    return leb_fail("leb_swiglu: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  LEB_CHECK_LAUNCH("leb_swiglu");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// out[p, :] = in[rows[p] / div, :]   (expert-sorted copies of token rows; div = experts per token)
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ in,
                                   const int* __restrict__ rows, int div, int D) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int p = blockIdx.x;
  int src = rows[p] / div;
  const T* a = in + (size_t)src * D;
  T* o = out + (size_t)p * D;
  if ((((uintptr_t)a | (uintptr_t)o) & 15) == 0 && (D * sizeof(T)) % 16 == 0) {
    const int n = D * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(a)[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = a[i];
  }
}

LEB_API int leb_gather_rows(void* out, const void* in, int dtype, const int* rows, int div, int P,
                            int D, cudaStream_t st) {
  if (P <= 0) return 0;
  LEB_REQUIRE(div >= 1, "leb_gather_rows: div must be positive");
  if (dtype == LEB_F32)
    leb_launch(gather_rows_kernel<float>, dim3(P), dim3(128), 0, st, (float*)out, (const float*)in, rows, div, D);
  else if (dtype == LEB_BF16)
    leb_launch(gather_rows_kernel<bf16>, dim3(P), dim3(128), 0, st, (bf16*)out, (const bf16*)in, rows, div, D);
  else
    return leb_fail("leb_gather_rows: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_gather_rows");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// x += y   (float residual; src/dense.rs:186,193)
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += y[i];
}
LEB_API int leb_add(float* x, const float* y, size_t n, cudaStream_t st) {
  if (n == 0) return 0;
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, y, n);
  LEB_CHECK_LAUNCH("leb_add");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// a[m, j] = act(gu[m, j]) * gu[m, F + j] with act chosen by code: 0 silu, 1 the tanh form of gelu,
// gelu(z) = z/2 * (1 + tanh(sqrt(2/pi) * (z + 0.044715 z^3))), 2 the clamped sigmoid form (below).
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
template <typename TI, typename TO>
__global__ void gated_act_kernel(TO* __restrict__ a, const TI* __restrict__ gu, int F, size_t total, int act,
                                 float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t m = i / F;
  int j = (int)(i - m * F);
  float g = to_f32(gu[m * 2 * F + j]);
  float u = to_f32(gu[m * 2 * F + F + j]);
  float r;
  if (act == 2) {        // clamped: g' = min(g, limit), u' = clamp(u, -limit, limit); g' sigmoid(alpha g') (u' + 1)
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    r = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
  } else {
    r = act == 1 ? gelu_tanh_f(g) * u : g / (1.0f + expf(-g)) * u;
  }
  a[i] = from_f32<TO>(r);
}

LEB_API int leb_gated_act(void* a, int out_dtype, const void* gu, int in_dtype, int M, int F, int act,
                          float limit, float alpha, cudaStream_t st) {
  size_t total = (size_t)M * F;
  if (total == 0) return 0;
  LEB_REQUIRE(act >= 0 && act <= 2, "leb_gated_act: unknown activation %d", act);
  LEB_REQUIRE(act != 2 || limit > 0.f, "leb_gated_act: the clamped activation needs a positive limit");
  dim3 grid((unsigned)((total + 255) / 256)), block(256);
  if (in_dtype == LEB_F32 && out_dtype == LEB_F32)
    leb_launch(gated_act_kernel<float, float>, grid, block, 0, st, (float*)a, (const float*)gu, F, total, act, limit, alpha);
  else if (in_dtype == LEB_F32 && out_dtype == LEB_BF16)
    leb_launch(gated_act_kernel<float, bf16>, grid, block, 0, st, (bf16*)a, (const float*)gu, F, total, act, limit, alpha);
  else if (in_dtype == LEB_BF16 && out_dtype == LEB_BF16)
    leb_launch(gated_act_kernel<bf16, bf16>, grid, block, 0, st, (bf16*)a, (const bf16*)gu, F, total, act, limit, alpha);
  else
    return leb_fail("leb_gated_act: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  LEB_CHECK_LAUNCH("leb_gated_act");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// The gated residual: x[m, i] += y[m, i] * sigmoid(z[m, i] + b[i]); x, y and b are float, the gate's
// pre-activation z comes from a matrix product in float or bfloat16 (row stride ldz: it may be a
// column range of a wider result).  Sum and sigmoid are float.  With `h` the same launch also
// leaves the RMS norm of the new row, h = x / sqrt(mean(x^2) + eps) * w, for the sublayer that reads
// the stream next (a block per row; the row is read back from cache for the second pass).
template <typename TZ, typename TH>
__global__ void __launch_bounds__(256) gated_residual_kernel(
    float* __restrict__ x, const float* __restrict__ y, const TZ* __restrict__ z, int ldz,
    const float* __restrict__ b, TH* __restrict__ h, const float* __restrict__ w, float eps, int D) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const size_t m = blockIdx.x;
  float* xr = x + m * D;
  const float* yr = y + m * D;
  const TZ* zr = z + m * ldz;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float zz = to_f32(zr[i]) + (b ? b[i] : 0.f);
    const float v = xr[i] + yr[i] * (1.0f / (1.0f + expf(-zz)));
    xr[i] = v;
    ss += v * v;
  }
  if (!h) return;
  ss = block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  TH* hr = h + m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) hr[i] = from_f32<TH>(xr[i] * r * w[i]);   // a thread re-reads what it wrote
}

// The same with 16-byte accesses for rows of up to CH * 512 * 4 elements: a thread keeps its pieces of the
// new row in registers between the sum and the norm, so a row is read once and a decode step's few
// rows are not a chain of dependent loads.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, c.x, c.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename TZ, typename TH, int CH>
__global__ void __launch_bounds__(512) gated_residual_vec_kernel(
    float* __restrict__ x, const float* __restrict__ y, const TZ* __restrict__ z, int ldz,
    const float* __restrict__ b, TH* __restrict__ h, const float* __restrict__ w, float eps, int D) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const size_t m = blockIdx.x;
  const int n4 = D >> 2;
  float4 v[CH];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < n4) {
      const float4 xv = load4(x + m * D + 4 * i), yv = load4(y + m * D + 4 * i), zv = load4(z + m * ldz + 4 * i);
      const float4 bv = b ? load4(b + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[c] = make_float4(xv.x + yv.x * sigmoid_f(zv.x + bv.x), xv.y + yv.y * sigmoid_f(zv.y + bv.y),
                         xv.z + yv.z * sigmoid_f(zv.z + bv.z), xv.w + yv.w * sigmoid_f(zv.w + bv.w));
      store4(x + m * D + 4 * i, v[c]);
      ss += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
    }
  }
  if (!h) return;
  ss = block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < n4) {
      const float4 wv = load4(w + 4 * i);
      store4(h + m * D + 4 * i, make_float4(v[c].x * r * wv.x, v[c].y * r * wv.y, v[c].z * r * wv.z, v[c].w * r * wv.w));
    }
  }
}

template <typename TZ, typename TH>
static void launch_gated_residual(float* x, const float* y, const void* z, int ldz, const float* b, void* h, const float* w,
                                  float eps, int M, int D, cudaStream_t st) {
  const int n4 = D / 4;
  const bool vec = D % 4 == 0 && n4 <= 4 * 512 && ldz % 4 == 0 && ((uintptr_t)z % (4 * sizeof(TZ))) == 0 &&
                   ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && (!b || ((uintptr_t)b % 16) == 0) &&
                   (!h || (((uintptr_t)h % (4 * sizeof(TH))) == 0 && ((uintptr_t)w % 16) == 0));
  if (vec) {
    const int ch = n4 <= 512 ? 1 : (n4 <= 1024 ? 2 : 4);
    const int threads = min(512, (ceil_div(n4, ch) + 31) / 32 * 32);
    if (ch == 1) leb_launch(gated_residual_vec_kernel<TZ, TH, 1>, dim3(M), dim3(threads), 0, st, x, y, (const TZ*)z, ldz, b, (TH*)h, w, eps, D);
    else if (ch == 2) leb_launch(gated_residual_vec_kernel<TZ, TH, 2>, dim3(M), dim3(threads), 0, st, x, y, (const TZ*)z, ldz, b, (TH*)h, w, eps, D);
    else leb_launch(gated_residual_vec_kernel<TZ, TH, 4>, dim3(M), dim3(threads), 0, st, x, y, (const TZ*)z, ldz, b, (TH*)h, w, eps, D);
    return;
  }
  leb_launch(gated_residual_kernel<TZ, TH>, dim3(M), dim3(D >= 1024 ? 256 : 128), 0, st, x, y, (const TZ*)z, ldz, b, (TH*)h, w, eps, D);
}

LEB_API int leb_gated_residual(float* x, const float* y, const void* z, int ldz, int z_dtype, const float* b, void* h,
                               int h_dtype, const float* w, float eps, int M, int D, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LEB_REQUIRE(!h || w, "leb_gated_residual: a norm needs its weight");
  // Launched strictly after its predecessor: with programmatic dependent launch a prompt step of several
  // thousand rows (a block per row here) now and then never finished on B200 -- one sequence of 8 x 2,000
  // rows in fifteen, never with these two kernels launched plainly; what waits on what was not found.
  LebPlainLaunches plain(true);
#define LEB_GR(TZ, TH) launch_gated_residual<TZ, TH>(x, y, z, ldz, b, h, w, eps, M, D, st)
  if (z_dtype == LEB_F32 && (!h || h_dtype == LEB_F32)) LEB_GR(float, float);
  else if (z_dtype == LEB_F32 && h_dtype == LEB_BF16) LEB_GR(float, bf16);
  else if (z_dtype == LEB_BF16 && (!h || h_dtype == LEB_BF16)) LEB_GR(bf16, bf16);
  else if (z_dtype == LEB_BF16 && h_dtype == LEB_F32) LEB_GR(bf16, float);
  else return leb_fail("leb_gated_residual: unknown dtypes z=%d h=%d", z_dtype, h_dtype);
#undef LEB_GR
  LEB_CHECK_LAUNCH("leb_gated_residual");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Additions to the residual stream between layers: x[m, :] += x0[m, :] (if given) + vec[:] (if given).
__global__ void stream_add_kernel(float* __restrict__ x, const float* __restrict__ x0,
                                  const float* __restrict__ vec, int D, size_t total) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i];
  if (x0) v += x0[i];
  if (vec) v += vec[i % D];
  x[i] = v;
}

LEB_API int leb_stream_add(float* x, const float* x0, const float* vec, int M, int D, cudaStream_t st) {
  size_t total = (size_t)M * D;
  if (total == 0 || (!x0 && !vec)) return 0;
  // Launched strictly after its predecessor: with programmatic dependent launch a prompt step of several
  // thousand rows (a block per row here) now and then never finished on B200 -- one sequence of 8 x 2,000
  // rows in fifteen, never with these two kernels launched plainly; what waits on what was not found.
  LebPlainLaunches plain(true);
  leb_launch(stream_add_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, x, x0, vec, D, total);
  LEB_CHECK_LAUNCH("leb_stream_add");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Layer norm with a weight and no bias: y = (x - mean) / sqrt(var + eps) * w, var the mean of the
// squared deviations (two passes over the row: the mean first, then the deviations).  All float.
//   rows != null : input row m is x[rows[m]]
template <typename TO>
__device__ __forceinline__ void layernorm_row(TO* __restrict__ o, const float* __restrict__ xi,
                                              const float* __restrict__ w, int D, float eps, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) s += xi[i];
  const float mean = block_sum(s, red) / (float)D;
  float v = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float d = xi[i] - mean;
    v += d * d;
  }
  const float r = 1.0f / sqrtf(block_sum(v, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = from_f32<TO>((xi[i] - mean) * r * w[i]);
}

template <typename TO>
__global__ void layernorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                 const int* __restrict__ rows, int D, float eps) {
  __shared__ float red[33];
  pdl_wait();
  const int m = blockIdx.x;
  layernorm_row(out + (size_t)m * D, x + (size_t)(rows ? rows[m] : m) * D, w, D, eps, red);
}

LEB_API int leb_layernorm(void* out, int out_dtype, const float* x, const float* w, const int* rows, int M, int D,
                          float eps, cudaStream_t st) {
  if (M <= 0) return 0;
  LebPlainLaunches plain(true);
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  if (out_dtype == LEB_F32) leb_launch(layernorm_kernel<float>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, rows, D, eps);
  else if (out_dtype == LEB_BF16) leb_launch(layernorm_kernel<bf16>, dim3(M), dim3(threads), 0, st, (bf16*)out, x, w, rows, D, eps);
  else return leb_fail("leb_layernorm: unknown output dtype %d", out_dtype);
  LEB_CHECK_LAUNCH("leb_layernorm");
  return 0;
}

// The sum of a layer whose sublayers read one norm: x[m, :] += mult * y[m, :] (y holds the sum of
// the sublayers' results), and with `h` the layer norm of the new row for whatever reads the
// stream next.  A thread re-reads only what it wrote.
template <typename TH>
__global__ void scaled_residual_kernel(float* __restrict__ x, const float* __restrict__ y, float mult,
                                       TH* __restrict__ h, const float* __restrict__ w, float eps, int D) {
  __shared__ float red[33];
  pdl_wait();
  const size_t m = blockIdx.x;
  float* xr = x + m * D;
  const float* yr = y + m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) xr[i] = xr[i] + mult * yr[i];
  if (!h) return;
  layernorm_row(h + m * D, xr, w, D, eps, red);
}

LEB_API int leb_scaled_residual(float* x, const float* y, float mult, void* h, int h_dtype, const float* w, float eps,
                                int M, int D, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LEB_REQUIRE(!h || w, "leb_scaled_residual: a norm needs its weight");
  LebPlainLaunches plain(true);
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  if (!h || h_dtype == LEB_F32)
    leb_launch(scaled_residual_kernel<float>, dim3(M), dim3(threads), 0, st, x, y, mult, (float*)h, w, eps, D);
  else if (h_dtype == LEB_BF16)
    leb_launch(scaled_residual_kernel<bf16>, dim3(M), dim3(threads), 0, st, x, y, mult, (bf16*)h, w, eps, D);
  else
    return leb_fail("leb_scaled_residual: unknown dtype %d", h_dtype);
  LEB_CHECK_LAUNCH("leb_scaled_residual");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Two layer norms of one row (weights w1 and w2, no bias): the mean and the variance are the row's, so
// they are formed once and both results written.  For layers whose sublayers each read the stream
// through a norm of their own.
template <typename TO>
__device__ __forceinline__ void layernorm_row2(TO* __restrict__ o1, TO* __restrict__ o2, const float* __restrict__ xi,
                                               const float* __restrict__ w1, const float* __restrict__ w2, int D,
                                               float eps, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) s += xi[i];
  const float mean = block_sum(s, red) / (float)D;
  float v = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float d = xi[i] - mean;
    v += d * d;
  }
  const float r = 1.0f / sqrtf(block_sum(v, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float t = (xi[i] - mean) * r;
    o1[i] = from_f32<TO>(t * w1[i]);
    o2[i] = from_f32<TO>(t * w2[i]);
  }
}

// x[m, :] += mult * y[m, :] when y is given; then the two layer norms of the (new) row.
template <typename TO>
__global__ void layernorm_pair_kernel(TO* __restrict__ h1, TO* __restrict__ h2, float* __restrict__ x,
                                      const float* __restrict__ y, float mult, const float* __restrict__ w1,
                                      const float* __restrict__ w2, int D, float eps) {
  __shared__ float red[33];
  pdl_wait();
  const size_t m = blockIdx.x;
  float* xr = x + m * D;
  if (y) {
    const float* yr = y + m * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) xr[i] = xr[i] + mult * yr[i];      // a thread re-reads only what it wrote
  }
  layernorm_row2(h1 + m * D, h2 + m * D, xr, w1, w2, D, eps, red);
}

LEB_API int leb_layernorm_pair(void* h1, void* h2, int dtype, float* x, const float* y, float mult, const float* w1,
                               const float* w2, int M, int D, float eps, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LebPlainLaunches plain(true);
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  if (dtype == LEB_F32)
    leb_launch(layernorm_pair_kernel<float>, dim3(M), dim3(threads), 0, st, (float*)h1, (float*)h2, x, y, mult, w1, w2, D, eps);
  else if (dtype == LEB_BF16)
    leb_launch(layernorm_pair_kernel<bf16>, dim3(M), dim3(threads), 0, st, (bf16*)h1, (bf16*)h2, x, y, mult, w1, w2, D, eps);
  else
    return leb_fail("leb_layernorm_pair: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_layernorm_pair");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// An activation without a gate, float in, the activation type out: 0 the erf form of gelu,
// z/2 (1 + erf(z / sqrt 2)); 1 the square of relu; 2 the tanh form of gelu; 3 silu.  x may be a column
// range of a wider result (row stride ldx).
template <typename TO>
__global__ void activation_kernel(TO* __restrict__ a, const float* __restrict__ x, int ldx, int F, size_t total, int act) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / F;
  const int j = (int)(i - m * F);
  const float z = x[m * ldx + j];
  float r;
  if (act == 0) r = 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));
  else if (act == 1) { const float t = fmaxf(z, 0.f); r = t * t; }
  else if (act == 2) r = gelu_tanh_f(z);
  else r = z / (1.0f + expf(-z));
  a[i] = from_f32<TO>(r);
}

LEB_API int leb_activation(void* a, int out_dtype, const float* x, int ldx, int M, int F, int act, cudaStream_t st) {
  const size_t total = (size_t)M * F;
  if (total == 0) return 0;
  LEB_REQUIRE(act >= 0 && act <= 3, "leb_activation: unknown activation %d", act);
  LebPlainLaunches plain(true);
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  if (out_dtype == LEB_F32) leb_launch(activation_kernel<float>, grid, block, 0, st, (float*)a, x, ldx, F, total, act);
  else if (out_dtype == LEB_BF16) leb_launch(activation_kernel<bf16>, grid, block, 0, st, (bf16*)a, x, ldx, F, total, act);
  else return leb_fail("leb_activation: unknown dtype %d", out_dtype);
  LEB_CHECK_LAUNCH("leb_activation");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Two sublayers' results side by side into one: out (+)= a (y1 + bias1) + b y2, all float [M, D];
// bias1 [D] or null.
__global__ void weighted_pair_sum_kernel(float* __restrict__ out, const float* __restrict__ y1, const float* __restrict__ bias1,
                                         float a, const float* __restrict__ y2, float b, int D, size_t total, int accumulate) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float l = y1[i] + (bias1 ? bias1[i % D] : 0.f);
  const float v = a * l + b * y2[i];
  out[i] = accumulate ? out[i] + v : v;
}

LEB_API int leb_weighted_pair_sum(float* out, const float* y1, const float* bias1, float a, const float* y2, float b, int M,
                                  int D, int accumulate, cudaStream_t st) {
  const size_t total = (size_t)M * D;
  if (total == 0) return 0;
  LebPlainLaunches plain(true);
  leb_launch(weighted_pair_sum_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, out, y1, bias1, a, y2, b, D,
             total, accumulate);
  LEB_CHECK_LAUNCH("leb_weighted_pair_sum");
  return 0;
}
