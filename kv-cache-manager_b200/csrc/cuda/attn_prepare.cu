// What lies between the q|k|v product of an attention mixer and the attention kernel, for mixers
// whose queries and keys are normalised, partly rotated or biased, and whose values may be mixed
// with an earlier layer's.  One block per row; the row stays in shared memory as floats:
//
//   1. proj row [q: nh*dk | k: nkv*dk | v: nkv*dv] (float) + bias (optional)
//   2. norm over the WHOLE q projection and over the whole k projection (optional):
//        q <- wq * q / sqrt(mean(q^2) + eps),  k likewise with wk
//   3. rotation of the first `rot` dimensions of every q and k head in rotate-half pairs
//        (i, i + rot/2), or with `interleaved` in neighbouring pairs (2i, 2i + 1),
//        angle = position * inv_freq[i]   (rot == 0: none)
//   4. norm per head, without weights (optional):  x <- x / sqrt(mean_head(x^2) + eps)
//   5. values: `v_keep` (optional, float [rows, nkv*dv]) receives v as projected;
//        `v_first` (optional, the same layout) mixes:  v <- v + lambda (v_first - v), evaluated as (1 - lambda) v + lambda v_first;
//        `v_inv_freq` (optional, dv/2 frequencies) turns every value head by its own position over all dv
//        dimensions, in the same pairing as q and k (what is cached is the turned value; the reader turns
//        the attention's output back by its own position)
//   6. q goes to q_out [rows, nh*HD] in the storage type, k and v to the row's page slot
//        [pages, nkv, page, HD]; HD >= max(dk, dv), elements beyond a head's own size are zero
//        (zeros add nothing to a score, and the attention output's columns beyond dv stay zero).
//
// With `maps` = M > 1 every query head and every key head holds M score maps side by side (the projection's
// q is nh*M*dk wide, head by head [map 0 | map 1 | ..], k is nkv*M*dk): bias, rotation and per-head norm work on
// each map's dk elements; q_out gets nh*M heads of HD, head h*M+m holding map m of query head h at elements
// [m*dk, (m+1)*dk) and zeros elsewhere; the key slot of head g holds its M maps one after another.  A query head
// of q_out therefore meets only its own map of the cached key, and the nh*M heads share the nkv key/value heads
// in the usual grouped way (M*dk <= HD).
//
// All arithmetic is float; the order of steps is the parameter list's, so a mixer that wants the
// norm before the rotation uses step 2 and one that wants it after uses step 4.
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

struct AttnPrepareParams {
  const float* proj; int ldp;
  const float* bias;                 // [nh*dk + nkv*dk + nkv*dv] or null
  const float* wq; const float* wk;  // weights of the whole-projection norm, or null (no such norm)
  const int* positions; const float* inv_freq; int rot;
  int head_norm;                     // 1: per-head norm without weights after the rotation
  float eps;
  float* v_keep; const float* v_first; const float* lambda;
  const int* slot_mapping; int block_size;
  void* q_out; void* k_cache; void* v_cache;
  int nh, nkv, dk, dv, HD;
  int interleaved;                   // pairs (2i, 2i+1) instead of (i, i + half)
  const float* v_inv_freq;           // [dv/2] or null
  int maps;                          // score maps per head (1: ordinary attention)
};

__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(512)
attn_prepare_kernel(AttnPrepareParams p) {
  extern __shared__ __align__(16) float row[];       // the row, then `rot` floats: cosines, sines
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int M = p.maps, nqu = p.nh * M, nku = p.nkv * M;         // units of dk elements: a map of a q or k head
  const int nq = nqu * p.dk, nk = nku * p.dk, nv = p.nkv * p.dv;
  const int n = nq + nk + nv;
  const int half = p.rot / 2;
  float* cs_table = row + n;
  float* vcs_table = cs_table + p.rot;               // dv floats: cosines, sines of the values' turn
  const int vhalf = p.v_inv_freq ? p.dv / 2 : 0;
  // the row's cosines and sines depend on nothing the step computes: before the wait
  if (half > 0 || vhalf > 0) {
    const float pos = float(p.positions[r]);
    for (int j = tid; j < half; j += blockDim.x) sincosf(pos * p.inv_freq[j], &cs_table[half + j], &cs_table[j]);
    for (int j = tid; j < vhalf; j += blockDim.x) sincosf(pos * p.v_inv_freq[j], &vcs_table[vhalf + j], &vcs_table[j]);
  }
  pdl_wait();
  const float* src = p.proj + size_t(r) * p.ldp;
  if ((n & 3) == 0 && (p.ldp & 3) == 0 && (reinterpret_cast<uintptr_t>(p.proj) & 15) == 0) {
    for (int i = 4 * tid; i < n; i += 4 * blockDim.x) {
      float4 v = *reinterpret_cast<const float4*>(src + i);
      if (p.bias) { v.x += p.bias[i]; v.y += p.bias[i + 1]; v.z += p.bias[i + 2]; v.w += p.bias[i + 3]; }
      *reinterpret_cast<float4*>(row + i) = v;
    }
  } else {
    for (int i = tid; i < n; i += blockDim.x) row[i] = src[i] + (p.bias ? p.bias[i] : 0.f);
  }
  __syncthreads();
  float iq = 1.f, ik = 1.f;
  if (p.wq) {                                        // the norm over the whole projections: the block's only reductions
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
    for (int i = tid; i < nk; i += blockDim.x) sk = fmaf(row[nq + i], row[nq + i], sk);
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    iq = 1.f / sqrtf(sq / float(nq) + p.eps);
    ik = 1.f / sqrtf(sk / float(nk) + p.eps);
  }
  // From here on a head is one warp's business: whole-projection scale, rotation, per-head norm, value
  // mixing and the store of that head need nothing of another head (two neighbouring elements a lane).
  const int slot = p.slot_mapping ? p.slot_mapping[r] : -1;
  const int page = slot >= 0 ? slot / p.block_size : 0, off = slot >= 0 ? slot - page * p.block_size : 0;
  const size_t base = (size_t(page) * p.nkv * p.block_size + off) * p.HD;
  const size_t head_stride = size_t(p.block_size) * p.HD;
  const float lam = p.v_first ? p.lambda[0] : 0.f;
  for (int u = warp; u < nqu + nku + p.nkv; u += nwarps) {
    if (u < nqu + nku) {                             // a query or key head (one map of it)
      const bool is_q = u < nqu;
      float* x = row + size_t(u) * p.dk;             // q heads, then k heads: both dk wide and adjacent
      if (p.wq) {
        const float inv = is_q ? iq : ik;
        const float* w = is_q ? p.wq + size_t(u) * p.dk : p.wk + size_t(u - nqu) * p.dk;
        for (int i = lane; i < p.dk; i += 32) x[i] = x[i] * inv * w[i];
        __syncwarp();
      }
      for (int j = lane; j < half; j += 32) {
        const int ia = p.interleaved ? 2 * j : j, ib = p.interleaved ? 2 * j + 1 : j + half;
        float a, b;
        rotate_pair(x[ia], x[ib], cs_table[j], cs_table[half + j], a, b);
        x[ia] = a;
        x[ib] = b;
      }
      __syncwarp();
      float inv = 1.f;
      if (p.head_norm) {
        float ss = 0.f;
        for (int i = lane; i < p.dk; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / float(p.dk) + p.eps);
      }
      T* dst;
      if (is_q) dst = reinterpret_cast<T*>(p.q_out) + (size_t(r) * nqu + u) * p.HD;
      else if (slot >= 0) dst = reinterpret_cast<T*>(p.k_cache) + base + ((u - nqu) / M) * head_stride;
      else continue;
      if (M == 1) {
        for (int d = 2 * lane; d < p.HD; d += 64)
          store_pair(dst + d, d < p.dk ? x[d] * inv : 0.f, d + 1 < p.dk ? x[d + 1] * inv : 0.f);
      } else {
        const int m = (is_q ? u : u - nqu) % M, lo = m * p.dk;
        if ((p.dk & 1) == 0) {                       // a map starts at an even element: two neighbours a store
          if (is_q) {                                // the whole padded head: the map at its place, zeros around it
            for (int d = 2 * lane; d < p.HD; d += 64) {
              const bool in = d >= lo && d < lo + p.dk;
              store_pair(dst + d, in ? x[d - lo] * inv : 0.f, in ? x[d - lo + 1] * inv : 0.f);
            }
          } else {                                   // this map's part of the key; the last map also the zeros behind
            for (int d = 2 * lane; d < p.dk; d += 64) store_pair(dst + lo + d, x[d] * inv, x[d + 1] * inv);
            if (m == M - 1)
              for (int d = M * p.dk + 2 * lane; d < p.HD; d += 64) store_pair(dst + d, 0.f, 0.f);
          }
        } else if (is_q) {
          for (int d = lane; d < p.HD; d += 32) stf(dst + d, d >= lo && d < lo + p.dk ? x[d - lo] * inv : 0.f);
        } else {
          for (int d = lane; d < p.dk; d += 32) stf(dst + lo + d, x[d] * inv);
          if (m == M - 1)
            for (int d = M * p.dk + lane; d < p.HD; d += 32) stf(dst + d, 0.f);
        }
      }
    } else {                                         // a value head
      const int head = u - nqu - nku;
      float* x = row + nq + nk + size_t(head) * p.dv;
      const size_t at = size_t(r) * nv + size_t(head) * p.dv;
      if (p.v_keep || p.v_first) {
        for (int i = lane; i < p.dv; i += 32) {
          const float v = x[i];
          if (p.v_keep) p.v_keep[at + i] = v;
          if (p.v_first) x[i] = (1.f - lam) * v + lam * p.v_first[at + i];
        }
        __syncwarp();
      }
      if (slot < 0) continue;
      if (vhalf > 0) {
        for (int j = lane; j < vhalf; j += 32) {
          const int ia = p.interleaved ? 2 * j : j, ib = p.interleaved ? 2 * j + 1 : j + vhalf;
          float a, b;
          rotate_pair(x[ia], x[ib], vcs_table[j], vcs_table[vhalf + j], a, b);
          x[ia] = a;
          x[ib] = b;
        }
        __syncwarp();
      }
      T* dst = reinterpret_cast<T*>(p.v_cache) + base + head * head_stride;
      for (int d = 2 * lane; d < p.HD; d += 64) store_pair(dst + d, d < p.dv ? x[d] : 0.f, d + 1 < p.dv ? x[d + 1] : 0.f);
    }
  }
}

template <typename T>
int launch_attn_prepare(const AttnPrepareParams& p, int rows, cudaStream_t s) {
  if (rows == 0) return 0;
  if (p.rot % 2 || p.rot > p.dk || p.maps < 1 || p.HD < p.maps * p.dk || p.HD < p.dv || p.HD % 2 || (p.v_inv_freq && p.dv % 2) ||
      (p.maps > 1 && p.wq))
    return KVCM_ERR_UNSUPPORTED;
  const size_t smem = size_t((p.nh + p.nkv) * p.maps * p.dk + p.nkv * p.dv + p.rot + (p.v_inv_freq ? p.dv : 0)) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(attn_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
  }
  // a row of a few thousand elements is a chain of short passes: more threads, fewer turns each
  const int threads = (p.nh * p.maps + 2 * p.nkv) * p.HD >= 2048 ? 512 : 256;
  return pdl_launch(attn_prepare_kernel<T>, dim3(rows), dim3(threads), smem, s, p);
}

}  // namespace kvcm

using namespace kvcm;

#define KVCM_ATTN_PREPARE_ARGS                                                                                        \
  const float *proj, int ldp, const float *bias, const float *wq, const float *wk, const int *positions,              \
      const float *inv_freq, int rot, int head_norm, float eps, float *v_keep, const float *v_first,                  \
      const float *lambda, const int *slot_mapping, int block_size, void *q_out, void *k_cache, void *v_cache,        \
      int rows, int nh, int nkv, int dk, int dv, int HD, int interleaved, const float *v_inv_freq, int maps, void *stream

static AttnPrepareParams make_params(KVCM_ATTN_PREPARE_ARGS) {
  (void)rows; (void)stream;
  AttnPrepareParams p;
  p.proj = proj; p.ldp = ldp; p.bias = bias; p.wq = wq; p.wk = wk; p.positions = positions; p.inv_freq = inv_freq;
  p.rot = inv_freq ? rot : 0; p.head_norm = head_norm; p.eps = eps; p.v_keep = v_keep; p.v_first = v_first; p.lambda = lambda;
  p.slot_mapping = slot_mapping; p.block_size = block_size; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.nh = nh; p.nkv = nkv; p.dk = dk; p.dv = dv; p.HD = HD; p.interleaved = interleaved; p.v_inv_freq = v_inv_freq; p.maps = maps;
  return p;
}

KVCM_API int kvcm_attn_prepare_f32(KVCM_ATTN_PREPARE_ARGS) {
  return launch_attn_prepare<float>(make_params(proj, ldp, bias, wq, wk, positions, inv_freq, rot, head_norm, eps, v_keep,
                                                v_first, lambda, slot_mapping, block_size, q_out, k_cache, v_cache, rows, nh,
                                                nkv, dk, dv, HD, interleaved, v_inv_freq, maps, stream), rows, (cudaStream_t)stream);
}
KVCM_API int kvcm_attn_prepare_bf16(KVCM_ATTN_PREPARE_ARGS) {
  return launch_attn_prepare<bf16>(make_params(proj, ldp, bias, wq, wk, positions, inv_freq, rot, head_norm, eps, v_keep,
                                               v_first, lambda, slot_mapping, block_size, q_out, k_cache, v_cache, rows, nh,
                                               nkv, dk, dv, HD, interleaved, v_inv_freq, maps, stream), rows, (cudaStream_t)stream);
}
