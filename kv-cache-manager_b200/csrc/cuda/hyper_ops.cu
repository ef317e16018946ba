// Several residual streams instead of one (hyper-connections), and what a differential attention mixer and a gated
// latent mixer need after their attention kernel.
//
//   embed_streams  x[row, s, :] = table[token[row]]  for every stream s                     (float32 streams)
//   hc_step        one pass over a row's S streams x[row, S, D] (float32, in place):
//                    write (optional, when a sublayer's output y is given):
//                        x'_t = sum_s mix[s, t] x_s + out[t] (y + bias)      all streams from the old ones
//                    read (optional, when an output is given):
//                        u = sum_s in[s] x'_s;   h = w * u / sqrt(mean(u^2) + eps)      (storage type)
//                  so the write that ends one sublayer and the read that opens the next are one kernel, also across
//                  layers and for the final norm (in = ones), which may gather the wanted rows only.  Sums run over
//                  s in ascending order: a row's result does not depend on the batch.
//   diff_combine   per row and head, from the two maps' attention outputs a1, a2 (heads 2h, 2h+1 of the attention
//                  kernel's output, padded heads of HD):  o = a1 - lambda a2;  o <- o / sqrt(mean(o^2) + eps) * post
//                  over the head's dv values;  o <- o * sigmoid(gate logit of the head);  storage type out
//   gate_mul       out = x * sigmoid(gate logits), element by element (gate logits float32 with a row stride)
//
// All arithmetic is float32 in both storage types.
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

constexpr int HC_MAX_STREAMS = 16;

template <typename W>
__global__ void __launch_bounds__(256)
embed_streams_kernel(const int* __restrict__ ids, const W* __restrict__ table, float* __restrict__ x, int S, int D, int vocab) {
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const W* src = table + size_t(id) * D;
  float* dst = x + size_t(row) * S * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = ldf(src + i);
    for (int s = 0; s < S; ++s) dst[size_t(s) * D + i] = v;
  }
}

struct HcParams {
  float* x;                 // [rows, S, D]
  const float* y;           // [rows, D] or null: nothing to write
  const float* bias;        // [D] or null
  const float* mix;         // [S, S], [from, to]
  const float* outw;        // [S]
  const float* inw;         // [S] or null: nothing to read
  const float* w;           // [D] norm weight
  void* h;                  // [n, D] storage type
  const int* rows;          // null, or the rows to work on (h has one row per index)
  int S, D;
  float eps;
};

template <typename T, int V, int MS>   // V columns a thread at a time (4: 16-byte accesses); at most MS streams
__global__ void __launch_bounds__(256, MS <= 4 ? 4 : 1)
hc_step_kernel(HcParams p) {
  extern __shared__ __align__(16) float hc_u[];          // D floats: the row's u
  __shared__ float coef[HC_MAX_STREAMS * HC_MAX_STREAMS + 2 * HC_MAX_STREAMS];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int S = p.S, D = p.D;
  float* mix = coef;
  float* outw = coef + S * S;
  float* inw = outw + S;
  // the coefficients are weights: nothing of the step writes them
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix[i] = p.y ? p.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    outw[i] = p.y ? p.outw[i] : 0.f;
    inw[i] = p.inw ? p.inw[i] : 0.f;
  }
  const int row = p.rows ? p.rows[blockIdx.x] : blockIdx.x;
  pdl_wait();
  __syncthreads();
  float* xr = p.x + size_t(row) * S * D;
  const float* yr = p.y ? p.y + size_t(row) * D : nullptr;
  float ss = 0.f;
  for (int d = V * threadIdx.x; d < D; d += V * blockDim.x) {
    float xs[MS][V];
#pragma unroll
    for (int s = 0; s < MS; ++s) {
      if (s < S) {
        if constexpr (V == 4) {
          const float4 a = *reinterpret_cast<const float4*>(xr + size_t(s) * D + d);
          xs[s][0] = a.x; xs[s][1] = a.y; xs[s][2] = a.z; xs[s][3] = a.w;
        } else {
          xs[s][0] = xr[size_t(s) * D + d];
        }
      }
    }
    if (yr) {
      float yv[V];
#pragma unroll
      for (int j = 0; j < V; ++j) yv[j] = yr[d + j] + (p.bias ? p.bias[d + j] : 0.f);
      float nx[MS][V];
#pragma unroll
      for (int t = 0; t < MS; ++t) {
        if (t < S) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MS; ++s)
              if (s < S) acc = fmaf(mix[s * S + t], xs[s][j], acc);
            nx[t][j] = fmaf(outw[t], yv[j], acc);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < MS; ++t) {
        if (t < S) {
#pragma unroll
          for (int j = 0; j < V; ++j) xs[t][j] = nx[t][j];
          if constexpr (V == 4) *reinterpret_cast<float4*>(xr + size_t(t) * D + d) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][3]);
          else xr[size_t(t) * D + d] = nx[t][0];
        }
      }
    }
    if (p.h) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < MS; ++s)
          if (s < S) u = fmaf(inw[s], xs[s][j], u);
        hc_u[d + j] = u;
        ss = fmaf(u, u, ss);
      }
    }
  }
  if (!p.h) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(D) + p.eps);
  T* dst = reinterpret_cast<T*>(p.h) + size_t(blockIdx.x) * D;
  for (int d = V * threadIdx.x; d < D; d += V * blockDim.x)
#pragma unroll
    for (int j = 0; j < V; ++j) stf(dst + d + j, p.w[d + j] * (hc_u[d + j] * inv));
}

template <typename T>
int launch_hc_step(const HcParams& p, int n, cudaStream_t s) {
  if (n == 0) return 0;
  if (p.S < 1 || p.S > HC_MAX_STREAMS || p.D < 1 || (!p.y && !p.h)) return KVCM_ERR_UNSUPPORTED;
  const size_t smem = size_t(p.D) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  const bool vec = (p.D & 3) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && p.S <= 8;   // registers: S x 4 x 2
  auto kernel = vec ? (p.S <= 2 ? hc_step_kernel<T, 4, 2> : p.S <= 4 ? hc_step_kernel<T, 4, 4> : hc_step_kernel<T, 4, 8>)
                    : (p.S <= 4 ? hc_step_kernel<T, 1, 4> : hc_step_kernel<T, 1, HC_MAX_STREAMS>);
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
  }
  const int per = vec ? 4 : 1;
  int threads = ((p.D + per - 1) / per + 31) / 32 * 32;
  threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
  return pdl_launch(kernel, dim3(n), dim3(threads), smem, s, p);
}

// One warp per (row, head).  a: [rows, 2*H heads of HD] (heads 2h and 2h+1 are the two maps of head h).  A lane holds
// four neighbouring elements at a time; heads of up to 512 values stay in registers between the sum of squares and the
// store (PER groups of four a lane), longer or odd ones are read a second time, element by element.
template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<bf16> {
  static __device__ __forceinline__ float2 load(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  static __device__ __forceinline__ void store(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};

template <typename T> struct Quad;                     // four neighbouring elements as floats
template <> struct Quad<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

template <typename T, int PER>
__global__ void __launch_bounds__(256)
diff_combine_kernel(const T* __restrict__ a, const float* __restrict__ gate, int ldg, const float* __restrict__ lambda,
                    T* __restrict__ out, int rows, int H, int dv, int HD, float eps, float post) {
  pdl_launch_dependents();
  const float lam = lambda[0];
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * H) return;
  const int row = unit / H, h = unit - row * H;
  const T* a1 = a + (size_t(row) * 2 * H + 2 * h) * HD;
  const T* a2 = a1 + HD;
  T* dst = out + (size_t(row) * H + h) * dv;
  float ss = 0.f;
  if constexpr (PER > 0) {                            // dv a multiple of 4, dv <= 128 * PER, 8- or 16-byte aligned rows
    float4 o[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = 4 * lane + 128 * i;
      o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d < dv) {
        const float4 x = Quad<T>::load(a1 + d), y = Quad<T>::load(a2 + d);
        o[i] = make_float4(fmaf(-lam, y.x, x.x), fmaf(-lam, y.y, x.y), fmaf(-lam, y.z, x.z), fmaf(-lam, y.w, x.w));
        ss = fmaf(o[i].x, o[i].x, fmaf(o[i].y, o[i].y, fmaf(o[i].z, o[i].z, fmaf(o[i].w, o[i].w, ss))));
      }
    }
    ss = warp_sum(ss);
    float f = post / sqrtf(ss / float(dv) + eps);
    if (gate) f *= 1.f / (1.f + expf(-gate[size_t(row) * ldg + h]));
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = 4 * lane + 128 * i;
      if (d < dv) Quad<T>::store(dst + d, make_float4(o[i].x * f, o[i].y * f, o[i].z * f, o[i].w * f));
    }
  } else {
    for (int d = lane; d < dv; d += 32) {
      const float o = fmaf(-lam, ldf(a2 + d), ldf(a1 + d));
      ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    float f = post / sqrtf(ss / float(dv) + eps);
    if (gate) f *= 1.f / (1.f + expf(-gate[size_t(row) * ldg + h]));
    for (int d = lane; d < dv; d += 32) stf(dst + d, fmaf(-lam, ldf(a2 + d), ldf(a1 + d)) * f);
  }
}

// out = x * sigmoid(gate): four neighbouring elements a thread where the rows allow 8- and 16-byte accesses.
template <typename T, int V>
__global__ void __launch_bounds__(256)
gate_mul_kernel(const T* __restrict__ x, const float* __restrict__ gate, int ldg, T* __restrict__ out, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const T* xr = x + size_t(row) * n;
  const float* gr = gate + size_t(row) * ldg;
  T* dst = out + size_t(row) * n;
  if constexpr (V == 4) {
    for (int i = 4 * threadIdx.x; i < n; i += 4 * blockDim.x) {
      const float4 g = *reinterpret_cast<const float4*>(gr + i);
      const float2 a = Pair<T>::load(xr + i), b = Pair<T>::load(xr + i + 2);
      Pair<T>::store(dst + i, a.x / (1.f + expf(-g.x)), a.y / (1.f + expf(-g.y)));
      Pair<T>::store(dst + i + 2, b.x / (1.f + expf(-g.z)), b.y / (1.f + expf(-g.w)));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) stf(dst + i, ldf(xr + i) / (1.f + expf(-gr[i])));
  }
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_embed_streams_f32(const int* ids, const void* table, float* x, int rows, int S, int D, int vocab, void* stream) {
  if (rows == 0) return 0;
  embed_streams_kernel<float><<<rows, 256, 0, (cudaStream_t)stream>>>(ids, (const float*)table, x, S, D, vocab);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_embed_streams_bf16(const int* ids, const void* table, float* x, int rows, int S, int D, int vocab, void* stream) {
  if (rows == 0) return 0;
  embed_streams_kernel<bf16><<<rows, 256, 0, (cudaStream_t)stream>>>(ids, (const bf16*)table, x, S, D, vocab);
  return KVCM_LAUNCH_RESULT();
}

#define KVCM_HC_STEP_ARGS                                                                                                 \
  float *x, const float *y, const float *bias, const float *mix, const float *outw, const float *inw, const float *w,     \
      void *h, const int *rows, int n, int S, int D, float eps, void *stream
static HcParams hc_params(KVCM_HC_STEP_ARGS) {
  (void)n; (void)stream;
  HcParams p;
  p.x = x; p.y = y; p.bias = bias; p.mix = mix; p.outw = outw; p.inw = inw; p.w = w; p.h = h; p.rows = rows;
  p.S = S; p.D = D; p.eps = eps;
  return p;
}
KVCM_API int kvcm_hc_step_f32(KVCM_HC_STEP_ARGS) {
  return launch_hc_step<float>(hc_params(x, y, bias, mix, outw, inw, w, h, rows, n, S, D, eps, stream), n, (cudaStream_t)stream);
}
KVCM_API int kvcm_hc_step_bf16(KVCM_HC_STEP_ARGS) {
  return launch_hc_step<bf16>(hc_params(x, y, bias, mix, outw, inw, w, h, rows, n, S, D, eps, stream), n, (cudaStream_t)stream);
}

#define KVCM_DIFF_COMBINE_ARGS                                                                                            \
  const void *a, const float *gate, int ldg, const float *lambda, void *out, int rows, int H, int dv, int HD, float eps, \
      float post, void *stream
template <typename T>
static int launch_diff_combine(KVCM_DIFF_COMBINE_ARGS) {
  if (rows == 0) return 0;
  if (H < 1 || dv < 1 || dv > HD) return KVCM_ERR_UNSUPPORTED;
  const int warps = 8, units = rows * H;
  const dim3 grid((units + warps - 1) / warps), block(warps * 32);
  const bool pairs = (dv & 3) == 0 && (HD & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
#define KVCM_DIFF(PER)                                                                                                    \
  return pdl_launch(diff_combine_kernel<T, PER>, grid, block, 0, (cudaStream_t)stream, (const T*)a, gate, ldg, lambda,    \
                    (T*)out, rows, H, dv, HD, eps, post)
  if (pairs && dv <= 128) KVCM_DIFF(1);
  if (pairs && dv <= 256) KVCM_DIFF(2);
  if (pairs && dv <= 512) KVCM_DIFF(4);
  KVCM_DIFF(0);
#undef KVCM_DIFF
}
KVCM_API int kvcm_diff_combine_f32(KVCM_DIFF_COMBINE_ARGS) {
  return launch_diff_combine<float>(a, gate, ldg, lambda, out, rows, H, dv, HD, eps, post, stream);
}
KVCM_API int kvcm_diff_combine_bf16(KVCM_DIFF_COMBINE_ARGS) {
  return launch_diff_combine<bf16>(a, gate, ldg, lambda, out, rows, H, dv, HD, eps, post, stream);
}

template <typename T>
static int launch_gate_mul(const void* x, const float* gate, int ldg, void* out, int rows, int n, void* stream) {
  if (rows == 0) return 0;
  const bool vec = (n & 3) == 0 && (ldg & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(gate) & 15) == 0;
  if (vec)
    return pdl_launch(gate_mul_kernel<T, 4>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const T*)x, gate, ldg, (T*)out, n);
  return pdl_launch(gate_mul_kernel<T, 1>, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (const T*)x, gate, ldg, (T*)out, n);
}
KVCM_API int kvcm_gate_mul_f32(const void* x, const float* gate, int ldg, void* out, int rows, int n, void* stream) {
  return launch_gate_mul<float>(x, gate, ldg, out, rows, n, stream);
}
KVCM_API int kvcm_gate_mul_bf16(const void* x, const float* gate, int ldg, void* out, int rows, int n, void* stream) {
  return launch_gate_mul<bf16>(x, gate, ldg, out, rows, n, stream);
}
