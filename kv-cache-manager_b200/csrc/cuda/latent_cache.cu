// A cache of one normalised vector per position (a compressed latent from which keys and values
// of all heads are expanded): c = w * v / sqrt(mean(v^2) + eps), statistics in float, written
// straight into the row's page slot.  The pages have the layout of the key pools,
// [pages, 1, page size, width], so the paged attention kernels read them as one shared head.
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_cache_kernel(const T* __restrict__ v, int ldv, const float* __restrict__ weight,
                         const int* __restrict__ slot_mapping, T* __restrict__ cache, int width, float eps) {
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const int slot = slot_mapping[row];
  if (slot < 0) return;                                   // a padding row holds no page
  const T* src = v + size_t(row) * ldv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float a = ldf(src + i);
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(width) + eps);
  T* dst = cache + size_t(slot) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) stf(dst + i, weight[i] * (ldf(src + i) * inv));
}


// The latent cache with a rotated part.  A row of `proj` (float) is [dq: qr | c: R | kr: dr]:
//   cq_out = T(wq * dq / rms(dq))                       the query's own latent (qr == 0: none)
//   page slot = [T(wc * c / rms(c)) : R | rotate(kr) : dr | zeros up to HD]
// kr is one key part shared by all heads: its first `rot` dimensions turn by position * inv_freq in pairs
// (2i, 2i+1) (`interleaved`) or (i, i + rot/2); it is not normalised.  Statistics, angles and the turn in float.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rope_cache_kernel(const float* __restrict__ proj, int ldp, const float* __restrict__ wq, const float* __restrict__ wc,
                         const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot, int interleaved,
                         const int* __restrict__ slot_mapping, T* __restrict__ cq_out, T* __restrict__ cache, int qr, int R,
                         int dr, int HD, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const float* src = proj + size_t(row) * ldp;
  // Both norms' sums are taken before the first barrier, so that all loads of the row are in flight together.
  const int slot = slot_mapping[row];
  const float* c = src + qr;
  float ssq = 0.f, ss = 0.f;
  for (int i = threadIdx.x; i < qr; i += blockDim.x) ssq = fmaf(src[i], src[i], ssq);
  if (slot >= 0)
    for (int i = threadIdx.x; i < R; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
  if (qr > 0) {
    ssq = block_sum(ssq, scratch);
    const float inv = 1.f / sqrtf(ssq / float(qr) + eps);
    for (int i = threadIdx.x; i < qr; i += blockDim.x) stf(cq_out + size_t(row) * qr + i, wq[i] * (src[i] * inv));
  }
  if (slot < 0) return;                                   // a padding row holds no page
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(R) + eps);
  T* dst = cache + size_t(slot) * HD;
  for (int i = threadIdx.x; i < R; i += blockDim.x) stf(dst + i, wc[i] * (c[i] * inv));
  const float* kr = c + R;
  const int half = rot / 2;
  const float pos = float(positions[row]);
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    float sn, cs, a, b;
    sincosf(pos * inv_freq[j], &sn, &cs);
    rotate_pair(kr[ia], kr[ib], cs, sn, a, b);
    stf(dst + R + ia, a);
    stf(dst + R + ib, b);
  }
  for (int i = rot + threadIdx.x; i < dr; i += blockDim.x) stf(dst + R + i, kr[i]);
  for (int i = R + dr + threadIdx.x; i < HD; i += blockDim.x) stf(dst + i, 0.f);
}

// The queries of the same mixer.  A row of `q` (float) holds per head [unrotated: dn | rotated: dr]:
//   qn_out[row, head, :] = T(unrotated part)                    (it goes on to the per-head map into the latent space)
//   qrow[row, head, R : R + dr] = rotate(rotated part);  qrow[row, head, R + dr : HD] = 0
// (qrow[row, head, 0 : R] is written by that map.)
template <typename T>
__global__ void __launch_bounds__(128)
latent_q_rope_kernel(const float* __restrict__ q, int ldq, const int* __restrict__ positions,
                     const float* __restrict__ inv_freq, int rot, int interleaved, T* __restrict__ qn_out,
                     T* __restrict__ qrow, int H, int dn, int dr, int R, int HD) {
  extern __shared__ __align__(16) float cs_table[];      // rot/2 cosines, rot/2 sines
  pdl_launch_dependents();
  const int row = blockIdx.x, half = rot / 2;
  const float pos = float(positions[row]);
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &cs_table[half + j], &cs_table[j]);
  pdl_wait();
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < H; h += nwarps) {
    const float* src = q + size_t(row) * ldq + size_t(h) * (dn + dr);
    T* qn = qn_out + (size_t(row) * H + h) * dn;
    for (int i = lane; i < dn; i += 32) stf(qn + i, src[i]);
    T* dst = qrow + (size_t(row) * H + h) * HD + R;
    const float* r = src + dn;
    for (int j = lane; j < half; j += 32) {
      const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
      float a, b;
      rotate_pair(r[ia], r[ib], cs_table[j], cs_table[half + j], a, b);
      stf(dst + ia, a);
      stf(dst + ib, b);
    }
    for (int i = rot + lane; i < dr; i += 32) stf(dst + i, r[i]);
    for (int i = dr + lane; i < HD - R; i += 32) stf(dst + i, 0.f);
  }
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_latent_norm_cache_f32(const void* v, int ldv, const float* weight, const int* slot_mapping,
                                        void* cache, int rows, int width, float eps, void* stream) {
  if (rows == 0) return 0;
  latent_norm_cache_kernel<float><<<rows, 128, 0, (cudaStream_t)stream>>>((const float*)v, ldv, weight, slot_mapping,
                                                                         (float*)cache, width, eps);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_latent_norm_cache_bf16(const void* v, int ldv, const float* weight, const int* slot_mapping,
                                         void* cache, int rows, int width, float eps, void* stream) {
  if (rows == 0) return 0;
  latent_norm_cache_kernel<bf16><<<rows, 128, 0, (cudaStream_t)stream>>>((const bf16*)v, ldv, weight, slot_mapping,
                                                                        (bf16*)cache, width, eps);
  return KVCM_LAUNCH_RESULT();
}

#define KVCM_LATENT_ROPE_CACHE_ARGS                                                                                   \
  const float *proj, int ldp, const float *wq, const float *wc, const int *positions, const float *inv_freq, int rot, \
      int interleaved, const int *slot_mapping, void *cq_out, void *cache, int rows, int qr, int R, int dr, int HD,  \
      float eps, void *stream
template <typename T>
static int launch_latent_rope_cache(KVCM_LATENT_ROPE_CACHE_ARGS) {
  if (rows == 0) return 0;
  if (rot % 2 || rot > dr || R + dr > HD || (qr > 0 && (!wq || !cq_out))) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(latent_rope_cache_kernel<T>, dim3(rows), dim3(128), 0, (cudaStream_t)stream, proj, ldp, wq, wc, positions,
                    inv_freq, rot, interleaved, slot_mapping, (T*)cq_out, (T*)cache, qr, R, dr, HD, eps);
}
KVCM_API int kvcm_latent_rope_cache_f32(KVCM_LATENT_ROPE_CACHE_ARGS) {
  return launch_latent_rope_cache<float>(proj, ldp, wq, wc, positions, inv_freq, rot, interleaved, slot_mapping, cq_out, cache,
                                         rows, qr, R, dr, HD, eps, stream);
}
KVCM_API int kvcm_latent_rope_cache_bf16(KVCM_LATENT_ROPE_CACHE_ARGS) {
  return launch_latent_rope_cache<bf16>(proj, ldp, wq, wc, positions, inv_freq, rot, interleaved, slot_mapping, cq_out, cache,
                                        rows, qr, R, dr, HD, eps, stream);
}

#define KVCM_LATENT_Q_ROPE_ARGS                                                                                     \
  const float *q, int ldq, const int *positions, const float *inv_freq, int rot, int interleaved, void *qn_out,    \
      void *qrow, int rows, int H, int dn, int dr, int R, int HD, void *stream
template <typename T>
static int launch_latent_q_rope(KVCM_LATENT_Q_ROPE_ARGS) {
  if (rows == 0) return 0;
  if (rot % 2 || rot > dr || R + dr > HD) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(latent_q_rope_kernel<T>, dim3(rows), dim3(128), size_t(rot) * sizeof(float), (cudaStream_t)stream, q, ldq,
                    positions, inv_freq, rot, interleaved, (T*)qn_out, (T*)qrow, H, dn, dr, R, HD);
}
KVCM_API int kvcm_latent_q_rope_f32(KVCM_LATENT_Q_ROPE_ARGS) {
  return launch_latent_q_rope<float>(q, ldq, positions, inv_freq, rot, interleaved, qn_out, qrow, rows, H, dn, dr, R, HD, stream);
}
KVCM_API int kvcm_latent_q_rope_bf16(KVCM_LATENT_Q_ROPE_ARGS) {
  return launch_latent_q_rope<bf16>(q, ldq, positions, inv_freq, rot, interleaved, qn_out, qrow, rows, H, dn, dr, R, HD, stream);
}
