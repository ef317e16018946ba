// A feed-forward made of many small gated experts of which every row uses a few.
//
//   route    router logits in float (one warp a row), softmax over all experts, optionally only the
//            experts of the best `keep` of `groups` equal groups of neighbours may be chosen (a
//            group's score is its largest expert score), the `top` largest scores win; a row's
//            weights are its chosen scores times `scale`, not renormalised.  An extra row of the
//            router matrix, if present, is a per-row gate: sigmoid of its logit.  Options: scores
//            sigmoid(z) instead of the softmax; a `correction` per expert that is added to the scores
//            for the choice only (choice scores may then be negative; the weights use the scores
//            themselves); a group's score as the sum of its two largest choice scores.
//   sort     the (row, choice) pairs ordered by expert, cut into tiles of 64 pairs of one expert.
//   gate_up  act[pair] = silu(h[row] Wg_e^T) * (h[row] Wu_e^T)      per tile, float accumulation
//   down     y[pair]   = act[pair] Wd_e^T                           per tile, float results
//   combine  out[row]  = sum_k weight[row, k] * y[row, k] + gate[row] * shared[row]   (float)
// (bfloat16 rows whose sizes allow it take the tensor-core form of the two products,
// csrc/cuda/moe_tcgen05.cu, after the same sort into tiles of 128.)
//
// Nothing is read on the host: counts and tile lists stay on the device and the product grids
// are sized for the worst case (pairs / 64 + experts tiles), so a step can be recorded into a
// CUDA graph.  Every output element is accumulated by one thread over k in ascending order, so
// a row's result does not depend on what else is in the batch or on the order inside a tile.
// Instantiated for float (the true 32-bit path: float FMAs only) and bfloat16 storage.
#include "common.cuh"

namespace kvcm {

constexpr int MOE_TM = 64, MOE_TN = 64, MOE_TK = 16;

__device__ __forceinline__ float moe_silu(float z) { return z / (1.f + expf(-z)); }

// (value, index) maximum over a warp; the lower index wins a tie.  Every lane gets the result.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// ------------------------------------------------------------------------------------ route
// One block of eight warps for RB rows: the rows of h are staged in shared memory as floats, the
// warps share out the experts (each logit one warp's sum over the width, float FMAs, 16-byte loads
// of the router's rows where they are aligned; a piece of the router's row is loaded once for all
// RB rows), then warp w does the softmax and the choice of rows w, w + 8, ...  RB = 1 for steps of
// few rows (more blocks), up to 8 for many (the router matrix is read once per block).
constexpr int ROUTE_WARPS = 8;
constexpr int ROUTE_EG = 4;      // experts a warp works on at a time

template <typename W> struct RouteVec;                     // elements of a 16-byte load
template <> struct RouteVec<float> { static constexpr int N = 4; };
template <> struct RouteVec<bf16> { static constexpr int N = 8; };

__device__ __forceinline__ void route_load(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
__device__ __forceinline__ void route_load(const bf16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __bfloat162float(h2[i].x); v[2 * i + 1] = __bfloat162float(h2[i].y); }
}

template <typename T, typename W, int RB>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, int ldh, const W* __restrict__ wr, int rows, int D, int E, int G, int keep,
                 int top, float scale, int has_gate, int vec_ok, int sigmoid_scores, const float* __restrict__ correction,
                 int group_top, int* __restrict__ idx, float* __restrict__ wt, float* __restrict__ gate_out) {
  extern __shared__ float route_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * RB;
  const int zstride = (2 * E + 1 + G + 3) & ~3;             // per row: scores, the gate's logit, the groups' scores, choice scores
  float* hs = route_smem + RB * zstride;                    // RB rows of h (16-byte aligned)
  for (int rr = 0; rr < RB; ++rr) {
    const bool live = row0 + rr < rows;
    const T* hr = h + size_t(live ? row0 + rr : row0) * ldh;
    for (int i = threadIdx.x; i < D; i += blockDim.x) hs[rr * D + i] = live ? ldf(hr + i) : 0.f;
  }
  __syncthreads();
  const int outs = E + (has_gate ? 1 : 0);
  constexpr int VN = RouteVec<W>::N;
  // A warp takes ROUTE_EG neighbouring experts at a time: a piece of the rows of h is read from shared
  // memory once for all of them, and their pieces of the router's rows are requested together.
  for (int e0 = warp * ROUTE_EG; e0 < outs; e0 += ROUTE_WARPS * ROUTE_EG) {
    float acc[ROUTE_EG][RB];
#pragma unroll
    for (int k = 0; k < ROUTE_EG; ++k)
#pragma unroll
      for (int rr = 0; rr < RB; ++rr) acc[k][rr] = 0.f;
    if (vec_ok) {
#pragma unroll 2
      for (int i = lane * VN; i < D; i += 32 * VN) {
        float v[ROUTE_EG][VN];
#pragma unroll
        for (int k = 0; k < ROUTE_EG; ++k)
          route_load(wr + size_t(min(e0 + k, outs - 1)) * D + i, v[k]);
#pragma unroll
        for (int rr = 0; rr < RB; ++rr) {
          float hv[VN];
#pragma unroll
          for (int j = 0; j < VN; j += 4) {
            const float4 a = *reinterpret_cast<const float4*>(hs + rr * D + i + j);
            hv[j] = a.x; hv[j + 1] = a.y; hv[j + 2] = a.z; hv[j + 3] = a.w;
          }
#pragma unroll
          for (int k = 0; k < ROUTE_EG; ++k)
#pragma unroll
            for (int j = 0; j < VN; ++j) acc[k][rr] = fmaf(hv[j], v[k][j], acc[k][rr]);
        }
      }
    } else {
      for (int i = lane; i < D; i += 32) {
        float v[ROUTE_EG];
#pragma unroll
        for (int k = 0; k < ROUTE_EG; ++k) v[k] = ldf(wr + size_t(min(e0 + k, outs - 1)) * D + i);
#pragma unroll
        for (int rr = 0; rr < RB; ++rr)
#pragma unroll
          for (int k = 0; k < ROUTE_EG; ++k) acc[k][rr] = fmaf(hs[rr * D + i], v[k], acc[k][rr]);
      }
    }
#pragma unroll
    for (int k = 0; k < ROUTE_EG; ++k)
#pragma unroll
      for (int rr = 0; rr < RB; ++rr) {
        const float a = warp_sum(acc[k][rr]);
        if (lane == 0 && e0 + k < outs) route_smem[rr * zstride + e0 + k] = a;
      }
  }
  __syncthreads();
  for (int rr = warp; rr < RB; rr += ROUTE_WARPS) {
    const int row = row0 + rr;
    if (row >= rows) break;
    float* z = route_smem + rr * zstride;
    float* gb = z + E + 1;
    float* ch = gb + G;                                        // choice scores: -inf once taken
    if (sigmoid_scores) {
      __syncwarp();
      for (int e = lane; e < E; e += 32) z[e] = 1.f / (1.f + expf(-z[e]));
    } else {
      float m = -INFINITY;
      for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
      m = warp_max(m);
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
      sum = warp_sum(sum);
      __syncwarp();
      for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - m) / sum;
    }
    for (int e = lane; e < E; e += 32) ch[e] = z[e] + (correction ? correction[e] : 0.f);
    if (has_gate && lane == 0) gate_out[row] = 1.f / (1.f + expf(-z[E]));
    __syncwarp();
    const int per = E / G;
    const bool limited = G > 1 && keep < G;
    if (limited) {
      for (int g = lane; g < G; g += 32) {
        float best = -INFINITY, second = -INFINITY;            // the group's two largest choice scores
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float c = ch[e];
          if (c > best) { second = best; best = c; }
          else if (c > second) second = c;
        }
        gb[g] = (group_top >= 2 && per >= 2) ? best + second : best;
      }
      __syncwarp();
      for (int k = 0; k < keep; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int g = lane; g < G; g += 32) {
          const float c = gb[g];
          if (c != INFINITY && (bi == 0x7fffffff || c > bv)) { bv = c; bi = g; }
        }
        warp_argmax(bv, bi);
        __syncwarp();
        if (lane == 0 && bi < G) gb[bi] = INFINITY;           // kept
        __syncwarp();
      }
    }
    for (int k = 0; k < top; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const bool allowed = !limited || gb[e / per] == INFINITY;
        const float c = ch[e];
        if (allowed && c != -INFINITY && (bi == 0x7fffffff || c > bv)) { bv = c; bi = e; }
      }
      warp_argmax(bv, bi);
      __syncwarp();
      if (lane == 0) {
        const bool ok = bi < E;
        idx[size_t(row) * top + k] = ok ? bi : 0;
        wt[size_t(row) * top + k] = ok ? z[bi] * scale : 0.f;
        if (ok) ch[bi] = -INFINITY;                            // taken
      }
      __syncwarp();
    }
  }
}

// ------------------------------------------------------------------------------------- sort
// One block.  offsets[e] = first sorted place of expert e; pair_of[place] = row * top + k and
// place_of[row * top + k] = place; tiles: (expert, first place, pairs) for every `tile_m` pairs of an
// expert; num_tiles[0] = how many.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int pairs, int E, int tile_m, int* __restrict__ offsets,
                int* __restrict__ pair_of, int* __restrict__ place_of, int* __restrict__ tile_expert,
                int* __restrict__ tile_begin, int* __restrict__ tile_rows, int* __restrict__ num_tiles) {
  extern __shared__ int sort_smem[];
  int* cnt = sort_smem;
  int* cursor = sort_smem + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      for (int b = 0; b < cnt[e]; b += tile_m, ++tiles) {
        tile_expert[tiles] = e;
        tile_begin[tiles] = at + b;
        tile_rows[tiles] = min(tile_m, cnt[e] - b);
      }
      at += cnt[e];
    }
    offsets[E] = at;
    num_tiles[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int place = atomicAdd(&cursor[idx[p]], 1);
    pair_of[place] = p;
    place_of[p] = place;
  }
}

// ----------------------------------------------------------------------------- the products
// act[place, n] = silu(sum_k h[row, k] Wg[e][n, k]) * (sum_k h[row, k] Wu[e][n, k]);
// wgu: [E, 2F, D], the F gate rows of an expert before its F up rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const T* __restrict__ h, int ldh, const T* __restrict__ wgu, const int* __restrict__ pair_of,
                   int top, const int* __restrict__ tile_expert, const int* __restrict__ tile_begin,
                   const int* __restrict__ tile_rows, const int* __restrict__ num_tiles, T* __restrict__ act,
                   int F, int D) {
  const int tile = blockIdx.y;
  if (tile >= num_tiles[0]) return;
  __shared__ float xs[MOE_TK][MOE_TM + 1];
  __shared__ float gsm[MOE_TK][MOE_TN + 1];
  __shared__ float usm[MOE_TK][MOE_TN + 1];
  __shared__ int src_row[MOE_TM];
  const int e = tile_expert[tile], begin = tile_begin[tile], mrows = tile_rows[tile];
  const int n0 = blockIdx.x * MOE_TN;
  const T* Wg = wgu + size_t(e) * 2 * F * D;
  const T* Wu = Wg + size_t(F) * D;
  if (threadIdx.x < MOE_TM) src_row[threadIdx.x] = threadIdx.x < mrows ? pair_of[begin + threadIdx.x] / top : -1;
  __syncthreads();
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float ag[4][4] = {}, au[4][4] = {};
  for (int k0 = 0; k0 < D; k0 += MOE_TK) {
    for (int i = threadIdx.x; i < MOE_TM * MOE_TK; i += 256) {
      const int r = i / MOE_TK, c = i % MOE_TK;
      const int src = src_row[r], gk = k0 + c;
      xs[c][r] = (src >= 0 && gk < D) ? ldf(h + size_t(src) * ldh + gk) : 0.f;
    }
    for (int i = threadIdx.x; i < MOE_TN * MOE_TK; i += 256) {
      const int r = i / MOE_TK, c = i % MOE_TK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < F && gk < D;
      gsm[c][r] = ok ? ldf(Wg + size_t(gn) * D + gk) : 0.f;
      usm[c][r] = ok ? ldf(Wu + size_t(gn) * D + gk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_TK; ++k) {
      float a[4], bg[4], bu[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { bg[j] = gsm[k][tx * 4 + j]; bu[j] = usm[k][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ag[i][j] = fmaf(a[i], bg[j], ag[i][j]);
          au[i][j] = fmaf(a[i], bu[j], au[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= mrows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < F) stf(act + size_t(begin + m) * F + gn, moe_silu(ag[i][j]) * au[i][j]);
    }
  }
}

// y[place, n] = sum_k act[place, k] Wd[e][n, k];  wd: [E, D, F];  y float, in the order of the sorted pairs.
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ wd, const int* __restrict__ tile_expert, const int* __restrict__ tile_begin,
                const int* __restrict__ tile_rows, const int* __restrict__ num_tiles, float* __restrict__ y,
                int F, int D) {
  const int tile = blockIdx.y;
  if (tile >= num_tiles[0]) return;
  __shared__ float xs[MOE_TK][MOE_TM + 1];
  __shared__ float ws[MOE_TK][MOE_TN + 1];
  const int e = tile_expert[tile], begin = tile_begin[tile], mrows = tile_rows[tile];
  const int n0 = blockIdx.x * MOE_TN;
  const T* W = wd + size_t(e) * D * F;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < F; k0 += MOE_TK) {
    for (int i = threadIdx.x; i < MOE_TM * MOE_TK; i += 256) {
      const int r = i / MOE_TK, c = i % MOE_TK;
      const int gk = k0 + c;
      xs[c][r] = (r < mrows && gk < F) ? ldf(act + size_t(begin + r) * F + gk) : 0.f;
    }
    for (int i = threadIdx.x; i < MOE_TN * MOE_TK; i += 256) {
      const int r = i / MOE_TK, c = i % MOE_TK;
      const int gn = n0 + r, gk = k0 + c;
      ws[c][r] = (gn < D && gk < F) ? ldf(W + size_t(gn) * F + gk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= mrows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < D) y[size_t(begin + m) * D + gn] = acc[i][j];
    }
  }
}

// out[row, i] = sum_k wt[row, k] * y[place_of[row * top + k], i]  (+ gate[row] * shared[row, i]),
// the choices added in the order of k.
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place_of, const float* __restrict__ wt, int top,
                   const float* __restrict__ shared_y, const float* __restrict__ gate, float* __restrict__ out, int D) {
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(wt[size_t(row) * top + k], y[size_t(place_of[size_t(row) * top + k]) * D + i], acc);
    if (shared_y) acc += (gate ? gate[row] : 1.f) * shared_y[size_t(row) * D + i];
    out[size_t(row) * D + i] = acc;
  }
}

template <typename T>
int launch_moe_route(const void* h, int ldh, const void* wr, int w_f32, int rows, int D, int E, int G, int keep, int top,
                     float scale, int has_gate, int sigmoid_scores, const float* correction, int group_top, int* idx,
                     float* wt, float* gate_out, cudaStream_t s) {
  if (rows == 0) return 0;
  if (E < 1 || G < 1 || E % G || keep < 1 || keep > G || top < 1 || top > (E / G) * keep || group_top < 1 || group_top > 2)
    return KVCM_ERR_UNSUPPORTED;
  const size_t zstride = (size_t(2 * E + 1 + G) + 3) & ~size_t(3);
  int rb = rows >= 512 ? 8 : 1;                                       // many rows: read the router once for 8 of them
  while (rb > 1 && (rb * (zstride + D)) * sizeof(float) > 160 * 1024) rb /= 2;
  const size_t smem = rb * (zstride + D) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  const int vec = w_f32 ? 4 : RouteVec<T>::N;
  const int vec_ok = (D % vec) == 0 && (reinterpret_cast<uintptr_t>(wr) & 15) == 0;
#define KVCM_ROUTE(W, RB)                                                                                             \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(moe_route_kernel<T, W, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    moe_route_kernel<T, W, RB><<<(rows + RB - 1) / RB, ROUTE_WARPS * 32, smem, s>>>(                                  \
        (const T*)h, ldh, (const W*)wr, rows, D, E, G, keep, top, scale, has_gate, vec_ok, sigmoid_scores, correction, \
        group_top, idx, wt, gate_out);                                                                                \
  } while (0)
#define KVCM_ROUTE_RB(W)                                                                                              \
  do {                                                                                                                \
    if (rb == 8) KVCM_ROUTE(W, 8);                                                                                    \
    else if (rb == 4) KVCM_ROUTE(W, 4);                                                                               \
    else if (rb == 2) KVCM_ROUTE(W, 2);                                                                               \
    else KVCM_ROUTE(W, 1);                                                                                            \
  } while (0)
  if (w_f32) KVCM_ROUTE_RB(float);
  else KVCM_ROUTE_RB(T);
#undef KVCM_ROUTE_RB
#undef KVCM_ROUTE
  return KVCM_LAUNCH_RESULT();
}

// The scratch of a step's routing, in ints: offsets[E + 1] | num_tiles[1] | pair_of[pairs] |
// place_of[pairs] | tile_expert, tile_begin, tile_rows [pairs / tile_m + E each].
struct MoeWork {
  int *offsets, *num_tiles, *pair_of, *place_of, *tile_expert, *tile_begin, *tile_rows;
  int max_tiles;
};
inline MoeWork moe_work(int* work, int pairs, int E, int tile_m) {
  MoeWork w;
  w.max_tiles = pairs / tile_m + E;
  w.offsets = work;
  w.num_tiles = work + E + 1;
  w.pair_of = w.num_tiles + 1;
  w.place_of = w.pair_of + pairs;
  w.tile_expert = w.place_of + pairs;
  w.tile_begin = w.tile_expert + w.max_tiles;
  w.tile_rows = w.tile_begin + w.max_tiles;
  return w;
}

int launch_moe_sort(const int* idx, int pairs, int E, int tile_m, int* work, cudaStream_t s) {
  if (size_t(2 * E) * sizeof(int) > 48 * 1024 || pairs / tile_m + E > 65535) return KVCM_ERR_UNSUPPORTED;
  const MoeWork w = moe_work(work, pairs, E, tile_m);
  moe_sort_kernel<<<1, 1024, size_t(2 * E) * sizeof(int), s>>>(idx, pairs, E, tile_m, w.offsets, w.pair_of, w.place_of,
                                                               w.tile_expert, w.tile_begin, w.tile_rows, w.num_tiles);
  return KVCM_LAUNCH_RESULT();
}

template <typename T>
int launch_moe_experts(const void* h, int ldh, const void* wgu, const void* wd, const int* idx, int rows, int top, int E,
                       int F, int D, int* work, void* act, float* y, cudaStream_t s) {
  if (rows == 0) return 0;
  const int pairs = rows * top;
  int rc = launch_moe_sort(idx, pairs, E, MOE_TM, work, s);
  if (rc) return rc;
  const MoeWork w = moe_work(work, pairs, E, MOE_TM);
  moe_gate_up_kernel<T><<<dim3((F + MOE_TN - 1) / MOE_TN, w.max_tiles), 256, 0, s>>>(
      (const T*)h, ldh, (const T*)wgu, w.pair_of, top, w.tile_expert, w.tile_begin, w.tile_rows, w.num_tiles, (T*)act, F, D);
  rc = KVCM_LAUNCH_RESULT();
  if (rc) return rc;
  moe_down_kernel<T><<<dim3((D + MOE_TN - 1) / MOE_TN, w.max_tiles), 256, 0, s>>>(
      (const T*)act, (const T*)wd, w.tile_expert, w.tile_begin, w.tile_rows, w.num_tiles, y, F, D);
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

// Ints of scratch that the experts' products need for `rows` rows (enough for tiles of 64 and of 128).
KVCM_API long long kvcm_moe_work_ints(int rows, int top, int E) {
  const long long pairs = (long long)rows * top;
  return (E + 2) + 2 * pairs + 3 * (pairs / MOE_TM + E);
}

// The tensor-core form of the experts' products (csrc/cuda/moe_tcgen05.cu), after a sort into tiles of 128.
extern "C" int kvcm_moe_experts_tcgen05_bf16(const void* h, int ldh, const void* wgu, const void* wd, const int* pair_of,
                                             const int* tile_expert, const int* tile_begin, const int* tile_rows,
                                             const int* num_tiles, int pairs, int top, int E, int F, int D, void* xs,
                                             void* act, float* y, void* stream);

// y in the order of the sorted pairs; `xs` [pairs, D] bf16 scratch.  Tensor-core products.
KVCM_API int kvcm_moe_experts_tc_bf16(const void* h, int ldh, const void* wgu, const void* wd, const int* idx, int rows,
                                      int top, int E, int F, int D, int* work, void* xs, void* act, float* y,
                                      void* stream) {
  if (rows == 0) return 0;
  const int pairs = rows * top;
  int rc = launch_moe_sort(idx, pairs, E, 128, work, (cudaStream_t)stream);
  if (rc) return rc;
  const MoeWork w = moe_work(work, pairs, E, 128);
  return kvcm_moe_experts_tcgen05_bf16(h, ldh, wgu, wd, w.pair_of, w.tile_expert, w.tile_begin, w.tile_rows, w.num_tiles,
                                       pairs, top, E, F, D, xs, act, y, stream);
}

#define KVCM_MOE(SUFFIX, T)                                                                                          \
  KVCM_API int kvcm_moe_route_##SUFFIX(const void* h, int ldh, const void* wr, int w_f32, int rows, int D, int E,    \
                                       int G, int keep, int top, float scale, int has_gate, int sigmoid_scores,      \
                                       const float* correction, int group_top, int* idx, float* wt,                  \
                                       float* gate_out, void* stream) {                                              \
    return launch_moe_route<T>(h, ldh, wr, w_f32, rows, D, E, G, keep, top, scale, has_gate, sigmoid_scores,         \
                               correction, group_top, idx, wt, gate_out, (cudaStream_t)stream);                      \
  }                                                                                                                  \
  KVCM_API int kvcm_moe_experts_##SUFFIX(const void* h, int ldh, const void* wgu, const void* wd, const int* idx,    \
                                         int rows, int top, int E, int F, int D, int* work, void* act, float* y,     \
                                         void* stream) {                                                             \
    return launch_moe_experts<T>(h, ldh, wgu, wd, idx, rows, top, E, F, D, work, act, y, (cudaStream_t)stream);      \
  }

KVCM_MOE(f32, float)
KVCM_MOE(bf16, bf16)

// `work` is the scratch the experts' products were given (it holds the place of every pair).
KVCM_API int kvcm_moe_combine(const float* y, const int* work, const float* wt, int top, int E, const float* shared_y,
                              const float* gate, float* out, int rows, int D, void* stream) {
  if (rows == 0) return 0;
  const int* place_of = work + E + 2 + rows * top;
  moe_combine_kernel<float><<<rows, 256, 0, (cudaStream_t)stream>>>(y, place_of, wt, top, shared_y, gate, out, D);
  return KVCM_LAUNCH_RESULT();
}
