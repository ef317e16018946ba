// Kernels of blocks whose sublayers are normalised on both sides (x <- x + post(sublayer(pre(x)))) and of
// the parts such designs bring along.  All arithmetic is float whatever the storage type T of the rows
// that go on to a matrix product; the residual stream x and every sublayer's output y are float.
//
//   embed_scaled    x[t] = table[id[t]] * scale (and a copy for parts that read the embedding later)
//   norm_post_pre   x += wb * y / rms(y)   (if y);   out = T(wn * x / rms(x))   (if out; optionally of gathered rows)
//                   -- the norm that closes one sublayer and the norm that opens the next in one pass
//   poly_norm_act   out = T(a N(z) + b N(z^2) + c N(z^3) + e), N(v) = v / rms(v) over a row, powers element-wise
//   concat_cast     out[t] = [T(a[t]) | T(b[t])]
//   add_bias_rows   x[t] += bias
//   softcap_rows    x <- cap * tanh(x / cap)
//   rotate_heads    turns pairs of the first `n` dimensions of every head of a row by sign * position * freq
//   gla_prepare     q *= qscale;  z <- sigmoid(z + bias)^(1/tau)  evaluated as exp(logsigmoid(z + bias) / tau)
//
// rms(v) = sqrt(mean(v^2) + eps).  Weights are given as the multipliers themselves, in float.
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

template <typename T>
__global__ void __launch_bounds__(256)
embed_scaled_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ x,
                    float* __restrict__ keep, int H, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + size_t(id) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = ldf(src + i) * scale;
    x[size_t(t) * H + i] = v;
    if (keep) keep[size_t(t) * H + i] = v;
  }
}

// One block a row; the row's new value stays in shared memory between the two passes.
template <typename T>
__global__ void __launch_bounds__(256)
norm_post_pre_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wb,
                     const float* __restrict__ wn, T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + size_t(r) * H;
  if (y) {
    const float* yr = y + size_t(r) * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = yr[i];
      row[i] = v;
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / float(H) + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = xr[i] + wb[i] * (row[i] * inv);
      row[i] = v;
      if (!rows) xr[i] = v;
      s2 = fmaf(v, v, s2);
    }
    if (!out) return;
    s2 = block_sum(s2, scratch);
    const float inv2 = 1.f / sqrtf(s2 / float(H) + eps);
    T* o = out + size_t(blockIdx.x) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) stf(o + i, wn[i] * (row[i] * inv2));
  } else {
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = xr[i];
      row[i] = v;
      s2 = fmaf(v, v, s2);
    }
    s2 = block_sum(s2, scratch);
    const float inv2 = 1.f / sqrtf(s2 / float(H) + eps);
    T* o = out + size_t(blockIdx.x) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) stf(o + i, wn[i] * (row[i] * inv2));
  }
}

// Four values a thread and access (H % 4 == 0 and 16-byte aligned rows); as many threads as a row has float4s, at most 512.
__device__ __forceinline__ void st4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void st4(bf16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&lo);
  u.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename T>
__global__ void __launch_bounds__(512)
norm_post_pre_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wb,
                         const float* __restrict__ wn, T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + size_t(r) * H;
  float s2 = 0.f;
  if (y) {
    const float* yr = y + size_t(r) * H;
    float ss = 0.f;
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(yr + i);
      *reinterpret_cast<float4*>(row + i) = v;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / float(H) + eps);
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + i), w = *reinterpret_cast<const float4*>(wb + i);
      float4 v = *reinterpret_cast<const float4*>(row + i);
      v.x = xv.x + w.x * (v.x * inv); v.y = xv.y + w.y * (v.y * inv);
      v.z = xv.z + w.z * (v.z * inv); v.w = xv.w + w.w * (v.w * inv);
      *reinterpret_cast<float4*>(row + i) = v;
      if (!rows) *reinterpret_cast<float4*>(xr + i) = v;
      s2 = fmaf(v.x, v.x, s2); s2 = fmaf(v.y, v.y, s2); s2 = fmaf(v.z, v.z, s2); s2 = fmaf(v.w, v.w, s2);
    }
    if (!out) return;
  } else {
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      *reinterpret_cast<float4*>(row + i) = v;
      s2 = fmaf(v.x, v.x, s2); s2 = fmaf(v.y, v.y, s2); s2 = fmaf(v.z, v.z, s2); s2 = fmaf(v.w, v.w, s2);
    }
  }
  s2 = block_sum(s2, scratch);
  const float inv2 = 1.f / sqrtf(s2 / float(H) + eps);
  T* o = out + size_t(blockIdx.x) * H;
  for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(row + i), w = *reinterpret_cast<const float4*>(wn + i);
    st4(o + i, w.x * (v.x * inv2), w.y * (v.y * inv2), w.z * (v.z * inv2), w.w * (v.w * inv2));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_act_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coef, T* __restrict__ out, int F,
                     float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* zr = z + size_t(blockIdx.x) * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = zr[i];
    row[i] = v;
    const float v2 = v * v, v3 = v2 * v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float n = float(F);
  const float a = coef[0] / sqrtf(s2 / n + eps), b = coef[1] / sqrtf(s4 / n + eps), c = coef[2] / sqrtf(s6 / n + eps);
  const float e = coef[3];
  T* o = out + size_t(blockIdx.x) * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = row[i], v2 = v * v;
    stf(o + i, a * v + b * v2 + c * (v2 * v) + e);
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
poly_norm_act_vec_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coef, T* __restrict__ out, int F,
                         float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* zr = z + size_t(blockIdx.x) * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = 4 * threadIdx.x; i < F; i += 4 * blockDim.x) {
    const float4 q = *reinterpret_cast<const float4*>(zr + i);
    *reinterpret_cast<float4*>(row + i) = q;
    const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float v2 = e[k] * e[k], v3 = v2 * e[k];
      s2 += v2;
      s4 = fmaf(v2, v2, s4);
      s6 = fmaf(v3, v3, s6);
    }
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float n = float(F);
  const float a = coef[0] / sqrtf(s2 / n + eps), b = coef[1] / sqrtf(s4 / n + eps), c = coef[2] / sqrtf(s6 / n + eps);
  const float e0 = coef[3];
  T* o = out + size_t(blockIdx.x) * F;
  for (int i = 4 * threadIdx.x; i < F; i += 4 * blockDim.x) {
    const float4 q = *reinterpret_cast<const float4*>(row + i);
    const float x2 = q.x * q.x, y2 = q.y * q.y, z2 = q.z * q.z, w2 = q.w * q.w;
    st4(o + i, a * q.x + b * x2 + c * (x2 * q.x) + e0, a * q.y + b * y2 + c * (y2 * q.y) + e0,
        a * q.z + b * z2 + c * (z2 * q.z) + e0, a * q.w + b * w2 + c * (w2 * q.w) + e0);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    stf(out + t * 2 * H + i, a[t * H + i]);
    stf(out + t * 2 * H + H + i, b[t * H + i]);
  }
}

__global__ void __launch_bounds__(256)
add_bias_rows_kernel(float* __restrict__ x, const float* __restrict__ bias, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) x[t * H + i] += bias[i];
}

__global__ void __launch_bounds__(256)
softcap_rows_kernel(float* __restrict__ x, long long n, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// One block a row, a warp a head at a time.
template <typename T>
__global__ void __launch_bounds__(128)
rotate_heads_kernel(T* __restrict__ x, int ldx, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                    int n, int interleaved, float sign, int nh, int HD) {
  extern __shared__ __align__(16) float cs[];        // n/2 cosines, n/2 sines
  pdl_launch_dependents();
  const int half = n / 2;
  const float pos = float(positions[blockIdx.x]);
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float sn, c;
    sincosf(pos * inv_freq[j], &sn, &c);
    cs[j] = c;
    cs[half + j] = sign * sn;
  }
  pdl_wait();
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < nh; h += nwarps) {
    T* v = x + size_t(blockIdx.x) * ldx + size_t(h) * HD;
    for (int j = lane; j < half; j += 32) {
      const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
      float a, b;
      rotate_pair(ldf(v + ia), ldf(v + ib), cs[j], cs[half + j], a, b);
      stf(v + ia, a);
      stf(v + ib, b);
    }
  }
}

// qkv rows [.. q: n_q floats at q_base ..]; z rows [heads*dk] become the decays.
__global__ void __launch_bounds__(256)
gla_prepare_kernel(float* __restrict__ qkv, int channels, int q_base, int n_q, float qscale, float* __restrict__ z,
                   const float* __restrict__ bias, int n_z, float inv_tau) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < n_q; i += blockDim.x) qkv[t * channels + q_base + i] *= qscale;
  for (int i = threadIdx.x; i < n_z; i += blockDim.x) {
    const float v = z[t * n_z + i] + (bias ? bias[i] : 0.f);
    const float ls = fminf(v, 0.f) - log1pf(expf(-fabsf(v)));      // log sigmoid(v)
    z[t * n_z + i] = expf(ls * inv_tau);
  }
}

}  // namespace kvcm

using namespace kvcm;

// Threads of a four-values-a-thread kernel over rows of n values: one float4 each, between 64 and 512.
static int vec_threads(int n) {
  const int t = ((n / 4) + 31) / 32 * 32;
  return t < 64 ? 64 : (t > 512 ? 512 : t);
}
template <typename... P>
static bool aligned16(const P*... p) {
  return (((reinterpret_cast<uintptr_t>(p)) | ...) & 15) == 0;
}

#define KVCM_EMBED_SCALED_ARGS const int *ids, const void *table, float *x, float *keep, int rows, int H, int vocab, float scale, void *stream
KVCM_API int kvcm_embed_scaled_f32(KVCM_EMBED_SCALED_ARGS) {
  if (rows == 0) return 0;
  return pdl_launch(embed_scaled_kernel<float>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, ids, (const float*)table, x,
                    keep, H, vocab, scale);
}
KVCM_API int kvcm_embed_scaled_bf16(KVCM_EMBED_SCALED_ARGS) {
  if (rows == 0) return 0;
  return pdl_launch(embed_scaled_kernel<bf16>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, ids, (const bf16*)table, x,
                    keep, H, vocab, scale);
}

template <typename T>
static int launch_norm_post_pre(float* x, const float* y, const float* wb, const float* wn, void* out, const int* rows_idx,
                                int rows, int H, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if ((y && !wb) || (out && !wn) || (!y && !out) || (rows_idx && !out)) return KVCM_ERR_UNSUPPORTED;
  const size_t smem = size_t(H) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  if (H % 4 == 0 && aligned16(x, y, wb, wn, out)) {
    if (smem > 40 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(norm_post_pre_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return int(e);
    }
    return pdl_launch(norm_post_pre_vec_kernel<T>, dim3(rows), dim3(vec_threads(H)), smem, s, x, y, wb, wn, (T*)out, rows_idx, H, eps);
  }
  if (smem > 40 * 1024) {                               // (the kernel's static shared memory counts against the 48 KB too)
    const cudaError_t e = cudaFuncSetAttribute(norm_post_pre_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
  }
  return pdl_launch(norm_post_pre_kernel<T>, dim3(rows), dim3(256), smem, s, x, y, wb, wn, (T*)out, rows_idx, H, eps);
}
#define KVCM_NORM_POST_PRE_ARGS float *x, const float *y, const float *wb, const float *wn, void *out, const int *rows_idx, int rows, int H, float eps, void *stream
KVCM_API int kvcm_norm_post_pre_f32(KVCM_NORM_POST_PRE_ARGS) {
  return launch_norm_post_pre<float>(x, y, wb, wn, out, rows_idx, rows, H, eps, (cudaStream_t)stream);
}
KVCM_API int kvcm_norm_post_pre_bf16(KVCM_NORM_POST_PRE_ARGS) {
  return launch_norm_post_pre<bf16>(x, y, wb, wn, out, rows_idx, rows, H, eps, (cudaStream_t)stream);
}

template <typename T>
static int launch_poly_norm(const float* z, int ldz, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  const size_t smem = size_t(F) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  if (F % 4 == 0 && ldz % 4 == 0 && aligned16(z, out)) {
    if (smem > 40 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(poly_norm_act_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return int(e);
    }
    return pdl_launch(poly_norm_act_vec_kernel<T>, dim3(rows), dim3(vec_threads(F)), smem, s, z, ldz, coef, (T*)out, F, eps);
  }
  if (smem > 40 * 1024) {                               // (the kernel's static shared memory counts against the 48 KB too)
    const cudaError_t e = cudaFuncSetAttribute(poly_norm_act_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
  }
  return pdl_launch(poly_norm_act_kernel<T>, dim3(rows), dim3(256), smem, s, z, ldz, coef, (T*)out, F, eps);
}
KVCM_API int kvcm_poly_norm_act_f32(const float* z, int ldz, const float* coef, void* out, int rows, int F, float eps, void* stream) {
  return launch_poly_norm<float>(z, ldz, coef, out, rows, F, eps, (cudaStream_t)stream);
}
KVCM_API int kvcm_poly_norm_act_bf16(const float* z, int ldz, const float* coef, void* out, int rows, int F, float eps, void* stream) {
  return launch_poly_norm<bf16>(z, ldz, coef, out, rows, F, eps, (cudaStream_t)stream);
}

KVCM_API int kvcm_concat_cast_f32(const float* a, const float* b, void* out, int rows, int H, void* stream) {
  if (rows == 0) return 0;
  return pdl_launch(concat_cast_kernel<float>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, a, b, (float*)out, H);
}
KVCM_API int kvcm_concat_cast_bf16(const float* a, const float* b, void* out, int rows, int H, void* stream) {
  if (rows == 0) return 0;
  return pdl_launch(concat_cast_kernel<bf16>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, a, b, (bf16*)out, H);
}

KVCM_API int kvcm_add_bias_rows(float* x, const float* bias, int rows, int H, void* stream) {
  if (rows == 0) return 0;
  return pdl_launch(add_bias_rows_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, x, bias, H);
}

KVCM_API int kvcm_softcap_rows(float* x, long long n, float cap, void* stream) {
  if (n == 0) return 0;
  if (!(cap > 0.f)) return KVCM_ERR_UNSUPPORTED;
  softcap_rows_kernel<<<unsigned((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, cap);
  return KVCM_LAUNCH_RESULT();
}

#define KVCM_ROTATE_HEADS_ARGS void *x, int ldx, const int *positions, const float *inv_freq, int n, int interleaved, float sign, int rows, int nh, int HD, void *stream
template <typename T>
static int launch_rotate_heads(KVCM_ROTATE_HEADS_ARGS) {
  if (rows == 0 || n == 0) return 0;
  if (n % 2 || n > HD) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(rotate_heads_kernel<T>, dim3(rows), dim3(128), size_t(n) * sizeof(float), (cudaStream_t)stream, (T*)x, ldx,
                    positions, inv_freq, n, interleaved, sign, nh, HD);
}
KVCM_API int kvcm_rotate_heads_f32(KVCM_ROTATE_HEADS_ARGS) {
  return launch_rotate_heads<float>(x, ldx, positions, inv_freq, n, interleaved, sign, rows, nh, HD, stream);
}
KVCM_API int kvcm_rotate_heads_bf16(KVCM_ROTATE_HEADS_ARGS) {
  return launch_rotate_heads<bf16>(x, ldx, positions, inv_freq, n, interleaved, sign, rows, nh, HD, stream);
}

KVCM_API int kvcm_gla_prepare(float* qkv, int channels, int q_base, int n_q, float qscale, float* z, const float* bias, int n_z,
                              float tau, int rows, void* stream) {
  if (rows == 0) return 0;
  if (!(tau > 0.f)) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(gla_prepare_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, qkv, channels, q_base, n_q, qscale, z,
                    bias, n_z, 1.f / tau);
}
