// The gated delta rule as a mixer with fixed-size state per request.
//
// Per value head (its query/key head is head / (heads / qk_heads)), with S a float matrix
// [dk, dv] that starts at zero and is carried from token to token:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// q, k, v come from projections that pass a short causal convolution over time per channel and
// SiLU; q and k are then scaled to unit length per head (q also by dk^-1/2); beta = sigmoid(b),
// g = exp(-exp(A_log) softplus(a + dt_bias)).  The head's output is divided by its root mean
// square, multiplied by a weight over dv and by SiLU of a gate projection.
//
// State of a request (one float slab per call site, `state_stride` floats a slot):
//     [ S: heads x dk x dv | last taps-1 inputs of the convolution: (taps-1) x channels ]
// Everything after the projections is float here, in both storage types.
//
// The columns of S are independent of each other, so the recurrence is spread over
// (request, head, 32 columns) blocks; inside a block four or eight lanes share a column (a run of
// neighbouring rows each) and add their partial dot products by shuffles.  The same kernel serves portions of
// prompts and single decoded tokens: it walks the request's rows of the step in order.  The
// recurrence is one dependent chain per column (dot product, step, update) whose length per token
// is what bounds a long portion of ONE request; requests and heads run side by side.
#include "common.cuh"

namespace kvcm {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ------------------------------------------------------------------ convolution over time + SiLU
// out[row, c] = silu( bias[c] + sum_j w[c, j] * in(local - (taps-1-j)) ) (bias optional), in(l) = this step's row l of the
// request when l >= 0, else what the state kept of earlier steps (zeros at the very start).
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_kernel(const T* __restrict__ proj, int ldp, const float* __restrict__ conv_w, int taps,
                  const float* __restrict__ state, long long state_stride, long long conv_off,
                  const int* __restrict__ row_seq, const int* __restrict__ seq_q_start,
                  const int* __restrict__ seq_state_slot, float* __restrict__ out, int channels,
                  const float* __restrict__ bias) {
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = row_seq[row];
  const int q0 = seq_q_start[s];
  const int slot = seq_state_slot[s];
  const int local = row - q0;
  const float* kept = slot >= 0 ? state + slot * state_stride + conv_off : nullptr;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int l = local - (taps - 1 - j);
    float v;
    if (l >= 0) v = ldf(proj + size_t(q0 + l) * ldp + c);
    else v = kept ? kept[size_t(taps - 1 + l) * channels + c] : 0.f;
    acc = fmaf(conv_w[size_t(c) * taps + j], v, acc);
  }
  out[size_t(row) * channels + c] = silu_f(acc);
}

// The same for up to kConvMaxTaps taps with every input read once: a thread owns one channel for a run of
// kConvRun consecutive rows and keeps the newest taps-1 inputs in registers (they are fetched as above where a
// request's rows begin inside the run).  The sum runs in the same order as above: the same bits.
constexpr int kConvMaxTaps = 8, kConvRun = 16;
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_run_kernel(const T* __restrict__ proj, int ldp, const float* __restrict__ conv_w, int taps,
                      const float* __restrict__ state, long long state_stride, long long conv_off,
                      const int* __restrict__ row_seq, const int* __restrict__ seq_q_start,
                      const int* __restrict__ seq_state_slot, float* __restrict__ out, int channels, int rows,
                      const float* __restrict__ bias) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int r0 = blockIdx.x * kConvRun, r1 = min(rows, r0 + kConvRun);
  float w[kConvMaxTaps], hist[kConvMaxTaps - 1];
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) w[j] = j < taps ? conv_w[size_t(c) * taps + j] : 0.f;
#pragma unroll
  for (int j = 0; j < kConvMaxTaps - 1; ++j) hist[j] = 0.f;
  const float b = bias ? bias[c] : 0.f;
  // the run's inputs and requests first, all loads in flight together; then the rows in order from registers
  float curv[kConvRun];
  int seqv[kConvRun];
#pragma unroll
  for (int i = 0; i < kConvRun; ++i) {
    const int row = r0 + i;
    seqv[i] = row < r1 ? row_seq[row] : -1;
    curv[i] = row < r1 ? ldf(proj + size_t(row) * ldp + c) : 0.f;
  }
  float wl = w[0];                                     // the current token's weight is the last tap's
#pragma unroll
  for (int j = 1; j < kConvMaxTaps; ++j) wl = (j == taps - 1) ? w[j] : wl;
  int prev_seq = -1;
#pragma unroll
  for (int i = 0; i < kConvRun; ++i) {
    const int row = r0 + i;
    if (row >= r1) break;
    const int s = seqv[i];
    if (s != prev_seq) {                               // a request's rows begin here (or the run does)
      prev_seq = s;
      const int q0 = seq_q_start[s], slot = seq_state_slot[s], local = row - q0;
      const float* kept = slot >= 0 ? state + slot * state_stride + conv_off : nullptr;
#pragma unroll
      for (int j = 0; j < kConvMaxTaps - 1; ++j) {
        if (j < taps - 1) {
          const int l = local - (taps - 1 - j);
          hist[j] = l >= 0 ? ldf(proj + size_t(q0 + l) * ldp + c) : (kept ? kept[size_t(taps - 1 + l) * channels + c] : 0.f);
        }
      }
    }
    const float cur = curv[i];
    float acc = b;
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 1; ++j)
      if (j < taps - 1) acc = fmaf(w[j], hist[j], acc);
    acc = fmaf(wl, cur, acc);
    out[size_t(row) * channels + c] = silu_f(acc);
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 2; ++j) hist[j] = hist[j + 1];
    // the newest input takes the place taps-2 (all places from there on hold it: only j < taps-1 is read)
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 1; ++j) hist[j] = (j >= taps - 2) ? cur : hist[j];
  }
}

// After the convolution has read it: the state keeps the last taps-1 inputs of each request.
// One thread owns one (request, channel) and moves old entries down before it overwrites them.
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(const T* __restrict__ proj, int ldp, int taps, float* __restrict__ state,
                        long long state_stride, long long conv_off, const int* __restrict__ seq_q_start,
                        const int* __restrict__ seq_q_len, const int* __restrict__ seq_state_slot, int channels) {
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = seq_state_slot[s];
  if (c >= channels || slot < 0) return;
  const int q0 = seq_q_start[s], n = seq_q_len[s];
  float* kept = state + slot * state_stride + conv_off;
  for (int j = 0; j < taps - 1; ++j) {
    const int l = n - (taps - 1) + j;
    const float v = l >= 0 ? ldf(proj + size_t(q0 + l) * ldp + c) : kept[size_t(n + j) * channels + c];
    kept[size_t(j) * channels + c] = v;
  }
}

// Both in one, for a step in which every request brings exactly one row (row == request): a thread owns one
// (request, channel), reads the kept inputs, writes the output and moves the state on.
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_single_kernel(const T* __restrict__ proj, int ldp, const float* __restrict__ conv_w, int taps,
                         float* __restrict__ state, long long state_stride, long long conv_off,
                         const int* __restrict__ seq_q_start, const int* __restrict__ seq_state_slot,
                         float* __restrict__ out, int channels, const float* __restrict__ bias) {
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int slot = seq_state_slot[s], row = seq_q_start[s];
  const float cur = ldf(proj + size_t(row) * ldp + c);
  float acc = bias ? bias[c] : 0.f;                   // summed in the order of the taps, as the general kernel does
  if (slot >= 0) {
    float* kept = state + slot * state_stride + conv_off;
    for (int j = 0; j < taps - 1; ++j) {
      const float v = kept[size_t(j) * channels + c];
      acc = fmaf(conv_w[size_t(c) * taps + j], v, acc);
      if (j > 0) kept[size_t(j - 1) * channels + c] = v;
    }
    if (taps > 1) kept[size_t(taps - 2) * channels + c] = cur;
  }
  acc = fmaf(conv_w[size_t(c) * taps + taps - 1], cur, acc);
  out[size_t(row) * channels + c] = silu_f(acc);
}

// ------------------------------------------------------------ unit vectors, step sizes, decays
// qkv[row]: the first 2 * qk_heads heads of dk (queries, then keys) become unit vectors
// (x / sqrt(sum x^2 + 1e-6); queries also times dk^-1/2).  ba[row] = [b | a] becomes [beta | g].
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ qkv, int channels, float* __restrict__ ba, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, int heads, int qk_heads, int dk) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float qscale = 1.f / sqrtf(float(dk));
  for (int hh = blockIdx.y * nwarps + warp; hh < 2 * qk_heads; hh += gridDim.y * nwarps) {
    float* p = qkv + size_t(row) * channels + size_t(hh) * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += p[i] * p[i];
    ss = warp_sum(ss);
    float inv = 1.f / sqrtf(ss + 1e-6f);
    if (hh < qk_heads) inv *= qscale;
    for (int i = lane; i < dk; i += 32) p[i] *= inv;
  }
  for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < heads; h += gridDim.y * blockDim.x) {
    float* r = ba + size_t(row) * 2 * heads;
    const float b = r[h];
    const float a = r[heads + h] + dt_bias[h];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    r[h] = 1.f / (1.f + expf(-b));
    r[heads + h] = expf(-expf(a_log[h]) * sp);
  }
}

// ------------------------------------------------------------------------------ the recurrence

// 4 bytes from global to shared memory without passing through registers; `ok` false writes zero.
__device__ __forceinline__ void dr_copy4(float* dst, const float* src, bool ok) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int bytes = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// 16 bytes (both addresses 16-byte aligned); `ok` false writes zeros.
__device__ __forceinline__ void dr_copy16(float* dst, const float* src, bool ok) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int bytes = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// DR_LANES lanes share a column; NI: rows of S per thread (dk <= DR_LANES * NI).  TT tokens are staged
// in shared memory at a time, in two buffers: while one tile of tokens is worked through, the next is
// on its way (cp.async).  Eight lanes a column for the longer keys: shorter chains of dependent FMAs
// per token and twice the warps to hide them behind.
// DR_COLS columns of S per block: 32, or fewer where that many blocks would leave SMs idle.
//
// MODE says which recurrence runs (the staging, the state and the split over blocks are the same):
//   kScanDelta        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q     one decay g per head
//   kScanDeltaChannel the same with channel-wise decays: row i of a head's S is scaled by gd[i]
//   kScanLinear       S <- g S + k (beta v)^T;  o = S^T q        (no correction by the state's own
//                     read-out: the selective state-space recurrence with k = B, q = C, beta = dt, v = x)
//   kScanLinearChannel  S <- diag(gd) S + k (beta v)^T;  o = S^T q   (the linear form with channel-wise decays:
//                     gated linear attention; `beta` may be null and then counts as one)
// Where q, k and v of a row lie is given by `q_base`, `k_base`, `v_base` (floats from the row's start).
struct ScanArgs {
  const float* qkv; int channels; int q_base, k_base, v_base;
  const float* beta; int beta_ld;        // [rows, >= heads]
  const float* g; int g_ld;              // [rows, >= heads]      (kScanDelta, kScanLinear)
  const float* gd;                       // [rows, heads * dk]    (kScanDeltaChannel)
  float* state; long long state_stride;
  const int* seq_q_start; const int* seq_q_len; const int* seq_state_slot;
  float* out; int heads, qk_heads, dk, dv;
};
constexpr int kScanDelta = 0, kScanDeltaChannel = 1, kScanLinear = 2, kScanLinearChannel = 3;

template <int DR_COLS, int DR_LANES, int NI, int TT, bool EARLY, int MODE>
__global__ void __launch_bounds__(DR_COLS * DR_LANES)
delta_scan_kernel(const ScanArgs A) {
  const float* __restrict__ qkv = A.qkv;
  const int channels = A.channels, heads = A.heads, qk_heads = A.qk_heads, dk = A.dk, dv = A.dv;
  float* __restrict__ state = A.state;
  const long long state_stride = A.state_stride;
  const int* __restrict__ seq_q_start = A.seq_q_start;
  const int* __restrict__ seq_q_len = A.seq_q_len;
  const int* __restrict__ seq_state_slot = A.seq_state_slot;
  float* __restrict__ out = A.out;
  constexpr bool CHD = MODE == kScanDeltaChannel || MODE == kScanLinearChannel;
  constexpr bool LIN = MODE == kScanLinear || MODE == kScanLinearChannel;
  constexpr int DKP = DR_LANES * NI;
  constexpr int CPW = 32 / DR_LANES;                      // columns per warp
  // A token's q and k lie in shared memory as in global memory, in 16-byte pieces (so that they are
  // staged by 16-byte copies), piece c at place c ^ (c / CH): lane r of a column owns the rows
  // r * NI .. r * NI + NI - 1 of S, i.e. the CH = NI / 4 pieces from r * CH on, and the exclusive-or
  // puts the pieces that the lanes of a warp read at the same time on different banks.
  // Elements from dk on stay zero.
  constexpr int CH = NI >= 8 ? NI / 4 : 1;
  auto place = [](int c) { return CH >= 2 ? (c ^ ((c / CH) & 7)) : c; };
  constexpr int NST = 2;                                  // tiles of tokens in shared memory or on their way
  __shared__ __align__(16) float qs[NST][TT][DKP];
  __shared__ __align__(16) float ks[NST][TT][DKP];
  __shared__ float vs[NST][TT][DR_COLS];
  __shared__ float bs[NST][TT], gs[NST][TT];
  __shared__ __align__(16) float gds[CHD ? NST : 1][CHD ? TT : 1][CHD ? DKP : 4];
  const int s = blockIdx.z, head = blockIdx.y;
  const int slot = seq_state_slot[s];
  const int q0 = seq_q_start[s], n = seq_q_len[s];
  if (slot < 0) {                                       // a padding entry: its rows of the output are zeros
    for (int idx = threadIdx.x; idx < n * DR_COLS; idx += blockDim.x) {
      const int c = blockIdx.x * DR_COLS + idx % DR_COLS;
      if (c < dv) out[size_t(q0 + idx / DR_COLS) * heads * dv + size_t(head) * dv + c] = 0.f;
    }
    return;
  }
  const int qk_head = head / (heads / qk_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_local = warp * CPW + (lane % CPW);
  const int col = blockIdx.x * DR_COLS + col_local;
  const int r = lane / CPW;
  const bool col_ok = col < dv;
  float* S = state + slot * state_stride + (size_t(head) * dk) * dv + col;
  float acc[NI];
#pragma unroll
  for (int m = 0; m < NI; ++m) {
    const int i = r * NI + m;
    acc[m] = (col_ok && i < dk) ? S[size_t(i) * dv] : 0.f;
  }
  for (int idx = threadIdx.x; idx < NST * TT * DKP; idx += blockDim.x) {
    (&qs[0][0][0])[idx] = 0.f;
    (&ks[0][0][0])[idx] = 0.f;
    if constexpr (CHD) (&gds[0][0][0])[idx] = 1.f;
  }
  __syncthreads();
  const size_t q_off = size_t(A.q_base) + size_t(qk_head) * dk, k_off = size_t(A.k_base) + size_t(qk_head) * dk;
  const size_t v_off = size_t(A.v_base) + size_t(head) * dv + size_t(blockIdx.x) * DR_COLS;
  const size_t gd_ld = size_t(heads) * dk, gd_off = size_t(head) * dk;
  const bool gvec16 = CHD && (dk % 4) == 0 && (reinterpret_cast<uintptr_t>(A.gd) & 15) == 0;
  const bool vec16 = (dk % 4) == 0 && (channels % 4) == 0 && (A.q_base % 4) == 0 && (A.k_base % 4) == 0 &&
                     (reinterpret_cast<uintptr_t>(qkv) & 15) == 0;

  // The 16-byte pieces of a tile are dealt out to the threads in the order (token, piece); a thread's first piece
  // and its step from one piece to its next are the same in every tile, so no loop below divides.
  const int per = max(dk / 4, 1);
  const int st_t0 = threadIdx.x / per, st_c0 = threadIdx.x % per, st_dt = blockDim.x / per, st_dc = blockDim.x % per;
  float* __restrict__ out_col = out + size_t(q0) * heads * dv + size_t(head) * dv + col;   // this column's outputs
  const size_t out_ld = size_t(heads) * dv;
  auto stage = [&](int buf, int t0) {                   // asks for the tile of tokens t0 .. t0 + TT - 1
    const int nt = min(TT, n - t0);
    if (vec16) {
      for (int t = st_t0, c = st_c0; t < TT; t += st_dt + (c + st_dc >= per), c = c + st_dc >= per ? c + st_dc - per : c + st_dc) {
        const bool ok = t < nt;
        const float* src = qkv + (ok ? size_t(q0 + t0 + t) * channels + 4 * c : 0);
        dr_copy16(&qs[buf][t][4 * place(c)], src + (ok ? q_off : 0), ok);
        dr_copy16(&ks[buf][t][4 * place(c)], src + (ok ? k_off : 0), ok);
      }
    } else {
      for (int idx = threadIdx.x; idx < TT * dk; idx += blockDim.x) {
        const int t = idx / dk, i = idx % dk;
        const bool ok = t < nt;
        const float* src = qkv + (ok ? size_t(q0 + t0 + t) * channels + i : 0);
        dr_copy4(&qs[buf][t][4 * place(i / 4) + i % 4], src + (ok ? q_off : 0), ok);
        dr_copy4(&ks[buf][t][4 * place(i / 4) + i % 4], src + (ok ? k_off : 0), ok);
      }
    }
    for (int idx = threadIdx.x; idx < TT * DR_COLS; idx += blockDim.x) {
      const int t = idx / DR_COLS, c = idx % DR_COLS;
      const bool ok = t < nt && blockIdx.x * DR_COLS + c < dv;
      dr_copy4(&vs[buf][t][c], qkv + (ok ? size_t(q0 + t0 + t) * channels + v_off + c : 0), ok);
    }
    for (int t = threadIdx.x; t < TT; t += blockDim.x) {
      const bool ok = t < nt;
      if (A.beta) dr_copy4(&bs[buf][t], A.beta + (ok ? size_t(q0 + t0 + t) * A.beta_ld + head : 0), ok);
      else bs[buf][t] = 1.f;
      if constexpr (!CHD) dr_copy4(&gs[buf][t], A.g + (ok ? size_t(q0 + t0 + t) * A.g_ld + head : 0), ok);
    }
    if constexpr (CHD) {
      if (gvec16) {
        for (int t = st_t0, c = st_c0; t < TT; t += st_dt + (c + st_dc >= per), c = c + st_dc >= per ? c + st_dc - per : c + st_dc) {
          const bool ok = t < nt;
          dr_copy16(&gds[buf][t][4 * place(c)], A.gd + (ok ? size_t(q0 + t0 + t) * gd_ld + gd_off + 4 * c : 0), ok);
        }
      } else {
        for (int idx = threadIdx.x; idx < TT * dk; idx += blockDim.x) {
          const int t = idx / dk, i = idx % dk;
          const bool ok = t < nt;
          dr_copy4(&gds[buf][t][4 * place(i / 4) + i % 4], A.gd + (ok ? size_t(q0 + t0 + t) * gd_ld + gd_off + i : 0), ok);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  stage(0, 0);
  for (int t0 = 0, buf = 0; t0 < n; t0 += TT, buf ^= 1) {
    const int nt = min(TT, n - t0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                                   // this tile has landed; the other buffer has been consumed
    if (t0 + TT < n) stage(buf ^ 1, t0 + TT);
    // One token: the state's step and the read-out.  `whole` false leaves the read-out as this lane's partial sum
    // (the caller adds the lanes of a column), so that the shuffles of several tokens can be in flight together.
    auto token = [&](int t, bool whole) -> float {
      const float g = CHD ? 1.f : gs[buf][t], beta = bs[buf][t];
      float kt[NI], qt[NI];
      if constexpr (CHD) {                            // the rows of S decay each by its own factor first
        if constexpr (NI % 4 == 0) {
#pragma unroll
          for (int m = 0; m < NI; m += 4) {
            const float4 d = *reinterpret_cast<const float4*>(&gds[buf][t][4 * place((r * NI + m) / 4)]);
            acc[m] *= d.x; acc[m + 1] *= d.y; acc[m + 2] *= d.z; acc[m + 3] *= d.w;
          }
        } else {
#pragma unroll
          for (int m = 0; m < NI; ++m) {
            const int i = r * NI + m;
            acc[m] *= gds[buf][t][4 * place(i / 4) + i % 4];
          }
        }
      }
      if constexpr (NI % 4 == 0) {
#pragma unroll
        for (int m = 0; m < NI; m += 4) {
          const int at = 4 * place((r * NI + m) / 4);
          const float4 a = *reinterpret_cast<const float4*>(&ks[buf][t][at]);
          const float4 b = *reinterpret_cast<const float4*>(&qs[buf][t][at]);
          kt[m] = a.x; kt[m + 1] = a.y; kt[m + 2] = a.z; kt[m + 3] = a.w;
          qt[m] = b.x; qt[m + 1] = b.y; qt[m + 2] = b.z; qt[m + 3] = b.w;
        }
      } else {
#pragma unroll
        for (int m = 0; m < NI; ++m) {
          const int i = r * NI + m, at = 4 * place(i / 4) + i % 4;
          kt[m] = ks[buf][t][at];
          qt[m] = qs[buf][t][at];
        }
      }
      float o;
      if constexpr (EARLY) {
        // Both read-outs are taken from the state BEFORE the token's write, so that neither waits for the
        // step u:  a = S^T k,  b = S^T q,  c = k . q;  u = beta (v - g a);  o = g b + c u  (= S_new^T q).
        // A shorter chain per token for a fifth more arithmetic: the form for few blocks.
        float a2[2] = {0.f, 0.f}, b2[2] = {0.f, 0.f}, c2[2] = {0.f, 0.f};
#pragma unroll
        for (int m = 0; m < NI; ++m) {
          a2[m & 1] = fmaf(acc[m], kt[m], a2[m & 1]);
          b2[m & 1] = fmaf(acc[m], qt[m], b2[m & 1]);
          c2[m & 1] = fmaf(kt[m], qt[m], c2[m & 1]);
        }
        float a = a2[0] + a2[1], b = b2[0] + b2[1], c = c2[0] + c2[1];
#pragma unroll
        for (int w = CPW; w < 32; w <<= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, w);
          b += __shfl_xor_sync(0xffffffffu, b, w);
          c += __shfl_xor_sync(0xffffffffu, c, w);
        }
        const float u = beta * (vs[buf][t][col_local] - g * a);
        o = fmaf(c, u, g * b);
#pragma unroll
        for (int m = 0; m < NI; ++m) acc[m] = fmaf(kt[m], u, g * acc[m]);
      } else {
        // In the order of the definition; four partial sums each keep the chains of dependent FMAs short.
        float u;
        if constexpr (LIN) {
          u = beta * vs[buf][t][col_local];
        } else {
          float p4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int m = 0; m < NI; ++m) p4[m & 3] = fmaf(acc[m], kt[m], p4[m & 3]);
          float p = (p4[0] + p4[1]) + (p4[2] + p4[3]);
#pragma unroll
          for (int w = CPW; w < 32; w <<= 1) p += __shfl_xor_sync(0xffffffffu, p, w);
          u = beta * (vs[buf][t][col_local] - g * p);
        }
        float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < NI; ++m) {
          acc[m] = fmaf(kt[m], u, g * acc[m]);
          o4[m & 3] = fmaf(acc[m], qt[m], o4[m & 3]);
        }
        o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        if (whole) {
#pragma unroll
          for (int w = CPW; w < 32; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
        }
      }
      return o;
    };
    int t = 0;
    if constexpr (LIN && !EARLY) {
      // The linear forms' step does not wait for the read-out: four tokens' read-outs are reduced side by side
      // (the same sums in the same order as one by one).
      for (; t + 4 <= nt; t += 4) {
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = token(t + j, false);
#pragma unroll
        for (int w = CPW; w < 32; w <<= 1) {
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] += __shfl_xor_sync(0xffffffffu, o[j], w);
        }
        if (r == 0 && col_ok) {
#pragma unroll
          for (int j = 0; j < 4; ++j) out_col[size_t(t0 + t + j) * out_ld] = o[j];
        }
      }
    }
#pragma unroll 1
    for (; t < nt; ++t) {
      const float o = token(t, true);
      if (r == 0 && col_ok) out_col[size_t(t0 + t) * out_ld] = o;
    }
  }
#pragma unroll
  for (int m = 0; m < NI; ++m) {
    const int i = r * NI + m;
    if (col_ok && i < dk) S[size_t(i) * dv] = acc[m];
  }
}

// --------------------------------------------------------------- gated norm of the heads' outputs
// out[row, h, j] = storage( o[row, h, j] / sqrt(mean_j o^2 + eps) * w[j] * silu(gate[row, h, j]) )
template <typename T>
__global__ void __launch_bounds__(128)
gated_rms_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ldg, const float* __restrict__ w,
                 T* __restrict__ out, int heads, int dv, float eps) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = blockIdx.y * nwarps + warp; h < heads; h += gridDim.y * nwarps) {
    const float* p = o + size_t(row) * heads * dv + size_t(h) * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss += p[j] * p[j];
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / float(dv) + eps);
    for (int j = lane; j < dv; j += 32) {
      const float gz = ldf(gate + size_t(row) * ldg + size_t(h) * dv + j);
      stf(out + size_t(row) * heads * dv + size_t(h) * dv + j, p[j] * inv * w[j] * silu_f(gz));
    }
  }
}

template <typename T>
int launch_delta_conv(const void* proj, int ldp, const float* conv_w, int taps, float* state, long long state_stride,
                      long long conv_off, const int* row_seq, const int* seq_q_start, const int* seq_q_len,
                      const int* seq_state_slot, float* out, int rows, int seqs, int channels, const float* bias,
                      cudaStream_t s) {
  if (rows == 0) return 0;
  if (taps < 1) return KVCM_ERR_UNSUPPORTED;
  const int by = (channels + 255) / 256;
  if (rows == seqs) {                            // every request brings one row: rows and requests coincide
    delta_conv_single_kernel<T><<<dim3(rows, by), 256, 0, s>>>((const T*)proj, ldp, conv_w, taps, state, state_stride, conv_off,
                                                               seq_q_start, seq_state_slot, out, channels, bias);
    return KVCM_LAUNCH_RESULT();
  }
  if (taps <= kConvMaxTaps)
    delta_conv_run_kernel<T><<<dim3((rows + kConvRun - 1) / kConvRun, by), 256, 0, s>>>(
        (const T*)proj, ldp, conv_w, taps, state, state_stride, conv_off, row_seq, seq_q_start, seq_state_slot, out, channels,
        rows, bias);
  else
    delta_conv_kernel<T><<<dim3(rows, by), 256, 0, s>>>((const T*)proj, ldp, conv_w, taps, state, state_stride, conv_off,
                                                        row_seq, seq_q_start, seq_state_slot, out, channels, bias);
  int rc = KVCM_LAUNCH_RESULT();
  if (rc || taps == 1) return rc;
  delta_conv_state_kernel<T><<<dim3(seqs, by), 256, 0, s>>>((const T*)proj, ldp, taps, state, state_stride, conv_off,
                                                            seq_q_start, seq_q_len, seq_state_slot, channels);
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_delta_conv_f32(const void* proj, int ldp, const float* conv_w, int taps, float* state,
                                 long long state_stride, long long conv_off, const int* row_seq,
                                 const int* seq_q_start, const int* seq_q_len, const int* seq_state_slot, float* out,
                                 int rows, int seqs, int channels, const float* bias, void* stream) {
  return launch_delta_conv<float>(proj, ldp, conv_w, taps, state, state_stride, conv_off, row_seq, seq_q_start,
                                  seq_q_len, seq_state_slot, out, rows, seqs, channels, bias, (cudaStream_t)stream);
}
KVCM_API int kvcm_delta_conv_bf16(const void* proj, int ldp, const float* conv_w, int taps, float* state,
                                  long long state_stride, long long conv_off, const int* row_seq,
                                  const int* seq_q_start, const int* seq_q_len, const int* seq_state_slot, float* out,
                                  int rows, int seqs, int channels, const float* bias, void* stream) {
  return launch_delta_conv<bf16>(proj, ldp, conv_w, taps, state, state_stride, conv_off, row_seq, seq_q_start,
                                 seq_q_len, seq_state_slot, out, rows, seqs, channels, bias, (cudaStream_t)stream);
}

KVCM_API int kvcm_delta_prepare(float* qkv, int channels, float* ba, const float* a_log, const float* dt_bias,
                                int rows, int heads, int qk_heads, int dk, void* stream) {
  if (rows == 0) return 0;
  const int by = (2 * qk_heads + 3) / 4;                       // a warp per query/key head, four to a block
  delta_prepare_kernel<<<dim3(rows, by), 128, 0, (cudaStream_t)stream>>>(qkv, channels, ba, a_log, dt_bias, heads, qk_heads, dk);
  return KVCM_LAUNCH_RESULT();
}

// Largest key size the recurrence kernel holds in registers.
KVCM_API int kvcm_delta_scan_max_dk() { return 256; }

// `rows`: rows of the step.  When every request brings one row (rows == seqs) the kernel is bound by
// reading and writing the state: four lanes a column then, so that a warp's access covers whole
// 32-byte sectors of a row of S.
template <int MODE>
static int launch_scan(const ScanArgs& A, int rows, int seqs, cudaStream_t s) {
  const int heads = A.heads, dk = A.dk, dv = A.dv;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  // 32 columns a block; 16 or 8 when that leaves SMs without a block (one request's long portion)
  const long long per32 = (long long)seqs * heads * ((dv + 31) / 32);
  // (the linear form with channel-wise decays is bound by its reads of shared memory, which narrower blocks
  // repeat: 16 columns at least)
  const int cols = per32 >= sms ? 32 : ((2 * per32 >= sms || MODE == kScanLinearChannel) ? 16 : 8);
  // few warps for the device (one request's long portion with few heads): the form with the shorter chain
  // (it has no meaning for the linear recurrence, whose step does not read the state)
  constexpr bool LIN = MODE == kScanLinear || MODE == kScanLinearChannel;
  constexpr bool CHD = MODE == kScanDeltaChannel || MODE == kScanLinearChannel;
  const bool early = !LIN && per32 * 8 <= 4LL * sms;
  // with a decay per channel a third staged array shares the static shared memory: fewer tokens a tile
  constexpr int TT_LONG = CHD ? 8 : 16, TT_LONGEST = CHD ? 4 : 8;
#define KVCM_SCAN_E(COLS, LANES, NI, TT, EARLY)                                                                     \
  delta_scan_kernel<COLS, LANES, NI, TT, EARLY, MODE><<<dim3((dv + COLS - 1) / COLS, heads, seqs), COLS * LANES, 0, s>>>(A)
#define KVCM_SCAN_C(COLS, LANES, NI, TT)                                                                            \
  do {                                                                                                              \
    if constexpr (LIN) KVCM_SCAN_E(COLS, LANES, NI, TT, false);                                                     \
    else if (early) KVCM_SCAN_E(COLS, LANES, NI, TT, true);                                                         \
    else KVCM_SCAN_E(COLS, LANES, NI, TT, false);                                                                   \
  } while (0)
#define KVCM_SCAN(LANES, NI, TT)                                                                                    \
  do {                                                                                                              \
    if (cols == 32) KVCM_SCAN_C(32, LANES, NI, TT);                                                                 \
    else if (cols == 16) KVCM_SCAN_C(16, LANES, NI, TT);                                                            \
    else KVCM_SCAN_C(8, LANES, NI, TT);                                                                             \
  } while (0)
  const bool single_rows = rows == seqs;
  if (dk <= 8) KVCM_SCAN(4, 2, 16);
  else if (dk <= 16) KVCM_SCAN(4, 4, 16);
  else if (dk <= 32) KVCM_SCAN(4, 8, 16);
  else if (dk <= 64) { if (single_rows) KVCM_SCAN(4, 16, 16); else KVCM_SCAN(8, 8, 16); }
  else if (dk <= 128) {
    if (single_rows) KVCM_SCAN(4, 32, TT_LONG);
    else if constexpr (MODE == kScanLinear) KVCM_SCAN(16, 8, 16);   // no chain through the step: more, shorter threads
    else KVCM_SCAN(8, 16, TT_LONG);
  }
  else KVCM_SCAN(8, 32, TT_LONGEST);
#undef KVCM_SCAN
#undef KVCM_SCAN_C
#undef KVCM_SCAN_E
  return KVCM_LAUNCH_RESULT();
}

// mode: 0 delta rule with one decay per head (g), 1 delta rule with a decay per head and key channel (gd),
// 2 linear recurrence, 3 linear recurrence with a decay per head and key channel (see the kernel).  The row layout of `qkv` is given by the three bases.
KVCM_API int kvcm_state_scan(int mode, const float* qkv, int channels, int q_base, int k_base, int v_base,
                             const float* beta, int beta_ld, const float* g, int g_ld, const float* gd, float* state,
                             long long state_stride, const int* seq_q_start, const int* seq_q_len,
                             const int* seq_state_slot, float* out, int rows, int seqs, int heads, int qk_heads, int dk,
                             int dv, void* stream) {
  if (seqs == 0) return 0;
  if (dk < 1 || dk > 256 || qk_heads < 1 || heads % qk_heads) return KVCM_ERR_UNSUPPORTED;
  const bool channel = mode == kScanDeltaChannel || mode == kScanLinearChannel;
  if (channel != (gd != nullptr) || (!channel && !g) || (!beta && mode != kScanLinearChannel)) return KVCM_ERR_UNSUPPORTED;
  ScanArgs A;
  A.qkv = qkv; A.channels = channels; A.q_base = q_base; A.k_base = k_base; A.v_base = v_base;
  A.beta = beta; A.beta_ld = beta_ld; A.g = g; A.g_ld = g_ld; A.gd = gd; A.state = state; A.state_stride = state_stride;
  A.seq_q_start = seq_q_start; A.seq_q_len = seq_q_len; A.seq_state_slot = seq_state_slot; A.out = out;
  A.heads = heads; A.qk_heads = qk_heads; A.dk = dk; A.dv = dv;
  cudaStream_t s = (cudaStream_t)stream;
  if (mode == kScanDelta) return launch_scan<kScanDelta>(A, rows, seqs, s);
  if (mode == kScanDeltaChannel) return launch_scan<kScanDeltaChannel>(A, rows, seqs, s);
  if (mode == kScanLinear) return launch_scan<kScanLinear>(A, rows, seqs, s);
  if (mode == kScanLinearChannel) return launch_scan<kScanLinearChannel>(A, rows, seqs, s);
  return KVCM_ERR_UNSUPPORTED;
}

// The delta rule with one decay per head: rows of `qkv` are [q | k | v], `bg` rows are [beta | g].
KVCM_API int kvcm_delta_scan(const float* qkv, int channels, const float* bg, float* state, long long state_stride,
                             const int* seq_q_start, const int* seq_q_len, const int* seq_state_slot, float* out,
                             int rows, int seqs, int heads, int qk_heads, int dk, int dv, void* stream) {
  return kvcm_state_scan(kScanDelta, qkv, channels, 0, qk_heads * dk, 2 * qk_heads * dk, bg, 2 * heads, bg + heads, 2 * heads,
                         nullptr, state, state_stride, seq_q_start, seq_q_len, seq_state_slot, out, rows, seqs, heads,
                         qk_heads, dk, dv, stream);
}

// ---------------------------------------------------- what the other recurrent mixers need around the scan

// Unit vectors as in delta_prepare; beta[row, h] = sigmoid(b[row, h]) (b in the storage type, row stride ldb);
// a[row, h, i] (float, in place) becomes the decay exp(-exp(A_log[h]) softplus(a + dt_bias[h, i])).
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_channel_kernel(float* __restrict__ qkv, int channels, const T* __restrict__ b, int ldb,
                             float* __restrict__ beta, float* __restrict__ a, const float* __restrict__ a_log,
                             const float* __restrict__ dt_bias, int heads, int qk_heads, int dk) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float qscale = 1.f / sqrtf(float(dk));
  for (int hh = blockIdx.y * nwarps + warp; hh < 2 * qk_heads; hh += gridDim.y * nwarps) {
    float* p = qkv + size_t(row) * channels + size_t(hh) * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += p[i] * p[i];
    ss = warp_sum(ss);
    float inv = 1.f / sqrtf(ss + 1e-6f);
    if (hh < qk_heads) inv *= qscale;
    for (int i = lane; i < dk; i += 32) p[i] *= inv;
  }
  for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < heads; h += gridDim.y * blockDim.x)
    beta[size_t(row) * heads + h] = 1.f / (1.f + expf(-ldf(b + size_t(row) * ldb + h)));
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < heads * dk; i += gridDim.y * blockDim.x) {
    const float z = a[size_t(row) * heads * dk + i] + dt_bias[i];
    const float sp = z > 20.f ? z : log1pf(expf(z));
    a[size_t(row) * heads * dk + i] = expf(-expf(a_log[i / dk]) * sp);
  }
}

// Step sizes and decays of the selective state-space recurrence: dt = softplus(raw + dt_bias) (no clamp),
// decay = exp(-exp(A_log) dt); out rows are [dt | decay].
template <typename T>
__global__ void __launch_bounds__(128)
ssm_prepare_kernel(const T* __restrict__ raw, int ld, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                   float* __restrict__ out, int rows, int heads) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * heads) return;
  const int row = idx / heads, h = idx - row * heads;
  const float z = ldf(raw + size_t(row) * ld + h) + dt_bias[h];
  const float dt = z > 20.f ? z : log1pf(expf(z));
  out[size_t(row) * 2 * heads + h] = dt;
  out[size_t(row) * 2 * heads + heads + h] = expf(-expf(a_log[h]) * dt);
}

// Norm of the recurrent mixers' outputs in groups of `group` neighbouring elements, with a gate:
//   v_i   = (o_i + skip_coef[i / head] * skip_i)  [* act(z_i) when the gate is applied ahead of the norm]
//   out_i = storage( v_i / sqrt(mean_group(v^2) + eps) * w[i % wlen]  [* act(z_i) when it comes after] )
// act: 0 = SiLU, 1 = sigmoid.  o float [rows, n]; z storage type (row stride ldz); skip float (row stride lds,
// optional, with one coefficient per `head` elements).  One warp per (row, group).
__device__ __forceinline__ float gate_act(float z, int act) {
  const float sg = 1.f / (1.f + expf(-z));
  return act == 0 ? z * sg : sg;
}
template <typename T>
__global__ void __launch_bounds__(128)
group_rms_gate_kernel(const float* __restrict__ o, const T* __restrict__ z, int ldz, const float* __restrict__ skip, int lds,
                      const float* __restrict__ skip_coef, int head, const float* __restrict__ w, int wlen,
                      T* __restrict__ out, int n, int group, int gate_first, int act, float eps) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int groups = n / group;
  for (int g = blockIdx.y * nwarps + warp; g < groups; g += gridDim.y * nwarps) {
    const int i0 = g * group;
    float ss = 0.f;
    for (int j = lane; j < group; j += 32) {
      const int i = i0 + j;
      float v = o[size_t(row) * n + i];
      if (skip) v = fmaf(skip_coef[i / head], skip[size_t(row) * lds + i], v);
      if (gate_first) v *= gate_act(ldf(z + size_t(row) * ldz + i), act);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / float(group) + eps);
    for (int j = lane; j < group; j += 32) {
      const int i = i0 + j;
      float v = o[size_t(row) * n + i];
      if (skip) v = fmaf(skip_coef[i / head], skip[size_t(row) * lds + i], v);
      const float gz = gate_act(ldf(z + size_t(row) * ldz + i), act);
      if (gate_first) v *= gz;
      v = v * inv * w[i % wlen];
      if (!gate_first) v *= gz;
      stf(out + size_t(row) * n + i, v);
    }
  }
}

// The same for groups of more than 256 elements: one block per (row, group), so that a long group's
// loads are in flight together instead of one warp walking it.
template <typename T>
__global__ void __launch_bounds__(256)
group_rms_gate_wide_kernel(const float* __restrict__ o, const T* __restrict__ z, int ldz, const float* __restrict__ skip,
                           int lds, const float* __restrict__ skip_coef, int head, const float* __restrict__ w, int wlen,
                           T* __restrict__ out, int n, int group, int gate_first, int act, float eps) {
  __shared__ float scratch[33];
  const int row = blockIdx.x, i0 = blockIdx.y * group;
  constexpr int kKeep = 8;                                 // values a thread keeps between the two passes
  float kept[kKeep], gates[kKeep];
  float ss = 0.f;
  int c = 0;
  for (int j = threadIdx.x; j < group; j += blockDim.x, ++c) {
    const int i = i0 + j;
    float v = o[size_t(row) * n + i];
    if (skip) v = fmaf(skip_coef[i / head], skip[size_t(row) * lds + i], v);
    const float gz = gate_act(ldf(z + size_t(row) * ldz + i), act);
    if (gate_first) v *= gz;
    if (c < kKeep) { kept[c] = v; gates[c] = gz; }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(group) + eps);
  c = 0;
  for (int j = threadIdx.x; j < group; j += blockDim.x, ++c) {
    const int i = i0 + j;
    float v, gz;
    if (c < kKeep) { v = kept[c]; gz = gates[c]; }
    else {
      v = o[size_t(row) * n + i];
      if (skip) v = fmaf(skip_coef[i / head], skip[size_t(row) * lds + i], v);
      gz = gate_act(ldf(z + size_t(row) * ldz + i), act);
      if (gate_first) v *= gz;
    }
    v = v * inv * w[i % wlen];
    if (!gate_first) v *= gz;
    stf(out + size_t(row) * n + i, v);
  }
}

template <typename T>
static int launch_group_rms_gate(const float* o, const void* z, int ldz, const float* skip, int lds, const float* skip_coef,
                                 int head, const float* w, int wlen, void* out, int rows, int n, int group, int gate_first,
                                 int act, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if (group < 1 || n % group || wlen < 1 || (skip && head < 1)) return KVCM_ERR_UNSUPPORTED;
  const int groups = n / group;
  if (group > 256 && groups <= 65535) {
    group_rms_gate_wide_kernel<T><<<dim3(rows, groups), 256, 0, s>>>(o, (const T*)z, ldz, skip, lds, skip_coef, head, w, wlen,
                                                                      (T*)out, n, group, gate_first, act, eps);
    return KVCM_LAUNCH_RESULT();
  }
  group_rms_gate_kernel<T><<<dim3(rows, (groups + 3) / 4), 128, 0, s>>>(o, (const T*)z, ldz, skip, lds, skip_coef, head, w, wlen,
                                                                       (T*)out, n, group, gate_first, act, eps);
  return KVCM_LAUNCH_RESULT();
}

#define KVCM_GROUP_RMS_ARGS                                                                                          \
  const float *o, const void *z, int ldz, const float *skip, int lds, const float *skip_coef, int head, const float *w, \
      int wlen, void *out, int rows, int n, int group, int gate_first, int act, float eps, void *stream
KVCM_API int kvcm_group_rms_gate_f32(KVCM_GROUP_RMS_ARGS) {
  return launch_group_rms_gate<float>(o, z, ldz, skip, lds, skip_coef, head, w, wlen, out, rows, n, group, gate_first, act, eps,
                                      (cudaStream_t)stream);
}
KVCM_API int kvcm_group_rms_gate_bf16(KVCM_GROUP_RMS_ARGS) {
  return launch_group_rms_gate<bf16>(o, z, ldz, skip, lds, skip_coef, head, w, wlen, out, rows, n, group, gate_first, act, eps,
                                     (cudaStream_t)stream);
}

KVCM_API int kvcm_delta_prepare_channel_f32(float* qkv, int channels, const void* b, int ldb, float* beta, float* a,
                                            const float* a_log, const float* dt_bias, int rows, int heads, int qk_heads,
                                            int dk, void* stream) {
  if (rows == 0) return 0;
  delta_prepare_channel_kernel<float><<<dim3(rows, max(1, min(16, (heads * dk + 511) / 512))), 128, 0, (cudaStream_t)stream>>>(qkv, channels, (const float*)b, ldb, beta, a,
                                                                              a_log, dt_bias, heads, qk_heads, dk);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_delta_prepare_channel_bf16(float* qkv, int channels, const void* b, int ldb, float* beta, float* a,
                                             const float* a_log, const float* dt_bias, int rows, int heads, int qk_heads,
                                             int dk, void* stream) {
  if (rows == 0) return 0;
  delta_prepare_channel_kernel<bf16><<<dim3(rows, max(1, min(16, (heads * dk + 511) / 512))), 128, 0, (cudaStream_t)stream>>>(qkv, channels, (const bf16*)b, ldb, beta, a,
                                                                             a_log, dt_bias, heads, qk_heads, dk);
  return KVCM_LAUNCH_RESULT();
}

KVCM_API int kvcm_ssm_prepare_f32(const void* raw, int ld, const float* a_log, const float* dt_bias, float* out, int rows,
                                  int heads, void* stream) {
  if (rows == 0) return 0;
  ssm_prepare_kernel<float><<<(rows * heads + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const float*)raw, ld, a_log, dt_bias,
                                                                                         out, rows, heads);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_ssm_prepare_bf16(const void* raw, int ld, const float* a_log, const float* dt_bias, float* out, int rows,
                                   int heads, void* stream) {
  if (rows == 0) return 0;
  ssm_prepare_kernel<bf16><<<(rows * heads + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const bf16*)raw, ld, a_log, dt_bias,
                                                                                        out, rows, heads);
  return KVCM_LAUNCH_RESULT();
}

KVCM_API int kvcm_gated_rms_f32(const float* o, const void* gate, int ldg, const float* w, void* out, int rows,
                                int heads, int dv, float eps, void* stream) {
  if (rows == 0) return 0;
  gated_rms_kernel<float><<<dim3(rows, (heads + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      o, (const float*)gate, ldg, w, (float*)out, heads, dv, eps);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_gated_rms_bf16(const float* o, const void* gate, int ldg, const float* w, void* out, int rows,
                                 int heads, int dv, float eps, void* stream) {
  if (rows == 0) return 0;
  gated_rms_kernel<bf16><<<dim3(rows, (heads + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      o, (const bf16*)gate, ldg, w, (bf16*)out, heads, dv, eps);
  return KVCM_LAUNCH_RESULT();
}
