// Mixers that carry a matrix of state per head from token to token, and the short causal convolutions in front of
// them.  Everything that enters a recurrence is float32: step sizes, decays, gates, unit norms, the state itself
// (step sizes and decays are taken in double and rounded to float32 once: a decay's error compounds over a sequence);
// the state of every sequence lies in float32 between steps and a step starts from what its slot holds.
//
//   causal_conv         y[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1) + j, c]) over the rows of one sequence;
//                       the rows before a step's first come from the slot's tail (the last taps - 1 inputs, zeros for
//                       a new sequence); a second kernel leaves the tail for the next step
//   selective_scan      per head, S [state, vdim]:  S = exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
//                       with dt = softplus(dt_raw + dt_bias); B and C are shared by the heads of a group
//   delta_rule_scan     per head, S [dim, vdim]:  S = diag(g) S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q
//                       with q, k unit vectors (q also times dim^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)),
//                       all of which delta_prepare makes ready for every token before the scan starts
//   decay_scan          per head, S [dim, vdim]:  S = a S + b k v^T;  o = S^T q, with one decay a a head and b = 1, or with
//                       a and b from exponential gates under a running maximum m (m' = max(f + m, i), a = exp(f + m - m'),
//                       b = exp(i - m')), a normalizer n = a n + b k and o = S^T q / (max(|n.q|, exp(-m')) + 1e-6);
//                       linear_prepare makes q, k, v float32 (an activation, a factor on q), exp_gates walks the maxima
//                       and leaves (a, b, exp(-m')) for every token; the scan carries n beside its state columns
//   gated_group_rmsnorm rows cut into groups, each divided by its own root mean square, times a weight; a gate
//                       multiplies either before the norm (silu) or after it (sigmoid)
//
// The scans walk a sequence's tokens in order: one thread block per (sequence, head, run of value columns); a thread
// holds a run of state rows of one, two or four value columns in registers; the tokens' vectors come through shared
// memory sixteen tokens at a time (cp.async, two stages), and the 8, 16 or 32 threads that share a column add their
// sums by shuffles.  The order of the sums does not depend on how a prompt was cut into steps or on what else is in
// the batch.  State layout: [slots, heads, vdim, rows] (the state's rows contiguous), so that a thread's part is one run.
#include "common.cuh"

// Kernels of a step may start while the kernel before them still runs (programmatic dependent launch); no pointer
// is declared __restrict__, and what the kernel right before wrote is read after griddepcontrol.wait.
namespace {
constexpr int CH = 16;      // tokens brought into shared memory at a time
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ double softplus_d(double v) { return v > 40.0 ? v : log1p(exp(v)); }

// ---- causal convolution ------------------------------------------------------------------------------
// x: rows of `stride` values (the convolved channels are its first `channels` from the pointer on); a block per
// (8 rows, run of channels), a thread per 4 channels (one where sizes or addresses do not allow 16-byte accesses)
// with the rows and its taps in registers
constexpr int CONV_TOKENS = 8, CONV_THREADS = 128;

template <int CPT> __device__ __forceinline__ void load_channels(const float* p, float (&v)[CPT]) {
  if constexpr (CPT == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int k = 0; k < CPT; ++k) v[k] = p[k];
  }
}
template <int CPT> __device__ __forceinline__ void load_channels(const __nv_bfloat16* p, float (&v)[CPT]) {
  if constexpr (CPT == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  } else {
#pragma unroll
    for (int k = 0; k < CPT; ++k) v[k] = __bfloat162float(p[k]);
  }
}

// A thread takes CPT consecutive channels of CONV_TOKENS consecutive rows; TMAX bounds the taps (4 or MAX_TAPS).
template <typename T, int CPT, int TMAX>
__global__ void __launch_bounds__(CONV_THREADS) causal_conv_kernel(const T* x, int stride, const float* w, const float* bias,
                                                                   const float* tail, const int* token_seq,
                                                                   const int* first_row, const int* slots, float* out,
                                                                   int n_tokens, int channels, int taps, int act,
                                                                   int n_seqs, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * CONV_TOKENS, c = (blockIdx.y * CONV_THREADS + threadIdx.x) * CPT;
  if (c >= channels) return;
  // everything the thread reads is asked for at once: the tile's rows and the taps - 1 before them, the taps, and
  // where each of the tile's tokens belongs
  float xs[CONV_TOKENS + TMAX - 1][CPT];  // xs[r]: row t0 - (taps - 1) + r
#pragma unroll
  for (int r = 0; r < CONV_TOKENS + TMAX - 1; ++r) {
    const int t = t0 - (taps - 1) + r;
    if (r < CONV_TOKENS + taps - 1 && t >= 0 && t < n_tokens) load_channels<CPT>(x + (size_t)t * stride + c, xs[r]);
    else {
#pragma unroll
      for (int k = 0; k < CPT; ++k) xs[r][k] = 0.f;
    }
  }
  float wt[CPT][TMAX], b[CPT];
#pragma unroll
  for (int k = 0; k < CPT; ++k) {
#pragma unroll
    for (int j = 0; j < TMAX; ++j) wt[k][j] = j < taps ? w[(size_t)(c + k) * taps + j] : 0.f;
    b[k] = bias ? bias[c + k] : 0.f;
  }
  int local[CONV_TOKENS], slot[CONV_TOKENS];
#pragma unroll
  for (int i = 0; i < CONV_TOKENS; ++i) {
    local[i] = -1;
    slot[i] = 0;
    if (t0 + i < n_tokens) {
      const int seq = token_seq[t0 + i];
      if (FMS_IN(seq, n_seqs)) {
        local[i] = t0 + i - first_row[seq];  // the row's place among its sequence's rows of this step
        slot[i] = __ldcg(slots + seq);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_TOKENS; ++i) {
    if (local[i] < 0 || !FMS_IN(slot[i], n_slots)) continue;
    const float* tl = tail + (size_t)slot[i] * (taps - 1) * channels;
    float acc[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k) acc[k] = b[k];
#pragma unroll
    for (int j = 0; j < TMAX; ++j) {
      if (j < taps) {
        const int back = taps - 1 - j;  // how many rows before this one
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
          const float v = back <= local[i] ? xs[i + j][k] : tl[(size_t)(taps - 1 + local[i] - back) * channels + c + k];
          acc[k] = fmaf(wt[k][j], v, acc[k]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < CPT; ++k) acc[k] = act ? acc[k] * sigmoid_f(acc[k]) : acc[k];
    float* o = out + (size_t)(t0 + i) * channels + c;
    if constexpr (CPT == 4) *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else {
#pragma unroll
      for (int k = 0; k < CPT; ++k) o[k] = acc[k];
    }
  }
}

// the tail after the step: the last taps - 1 inputs of (old tail, the step's rows); one thread per (sequence, channel)
template <typename T>
__global__ void conv_tail_kernel(const T* x, int stride, float* tail, const int* first_row, const int* slots,
                                 int channels, int taps, int n_seqs, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
  if (c >= channels) return;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], n = first_row[seq + 1] - lo;
  float* tl = tail + (size_t)slot * (taps - 1) * channels;
  float keep[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps - 1) break;
    const int local = n - (taps - 1) + j;
    keep[j] = local >= 0 ? to_f32(x[(size_t)(lo + local) * stride + c]) : tl[(size_t)(j + n) * channels + c];
  }
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps - 1) break;
    tl[(size_t)j * channels + c] = keep[j];
  }
}

// ---- the two scans ------------------------------------------------------------------------------------
// Both walk a sequence's tokens in order with the state in registers.  A block of 128 threads owns (sequence, head,
// run of VB = 16 * VP value columns); a thread owns VP columns and NP consecutive state rows of each, and the eight
// (or 16, or 32: PARTS) threads that share a column group add their sums by shuffles, so a column's sum runs over its rows in the
// same order whatever VP is, whatever else is in the batch and however the prompt was cut.  The tokens' vectors
// come through shared memory CH tokens at a time by cp.async into two stages: the next chunk is on its way while this
// one is walked.  Rows of shared memory are padded to PARTS * NP values with zeros, so the inner loops need no bounds.
constexpr int SCAN_THREADS = 128;  // PARTS threads share a group of value columns; a block has 128 / PARTS groups

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// rows of `count` floats from global rows (stride src_stride) into shared rows (stride dst_stride), `rows` of them;
// 16 bytes a copy where `vec` says that every row's start and length allow it
__device__ __forceinline__ void stage_rows(float* dst, int dst_stride, const float* src, size_t src_stride, int rows,
                                           int count, bool vec) {
  if (vec) {
    const int per = count >> 2;
    for (int i = threadIdx.x; i < rows * per; i += blockDim.x) {
      const int r = i / per, c = (i - r * per) << 2;
      cp_async16(dst + r * dst_stride + c, src + r * src_stride + c);
    }
  } else {
    for (int i = threadIdx.x; i < rows * count; i += blockDim.x) {
      const int r = i / count, c = i - r * count;
      cp_async4(dst + r * dst_stride + c, src + r * src_stride + c);
    }
  }
}

// A row of shared memory holds PARTS runs of NP values, one per thread of a column group.  From NP = 8 on the runs lie
// NP + 4 values apart, so that the eight 16-byte loads of a group's threads fall into different banks.
template <int NP, int PARTS> struct RowLayout {
  static constexpr int RUN = NP >= 8 ? NP + 4 : NP;
  static constexpr int ROW = PARTS * RUN;
  __device__ static __forceinline__ int at(int n) { return (n / NP) * RUN + (n % NP); }
};
template <int NP> __device__ __forceinline__ void load_run(const float* p, float (&r)[NP]) {
  if constexpr (NP % 4 == 0) {
#pragma unroll
    for (int j = 0; j < NP; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + j);
      r[j] = v.x; r[j + 1] = v.y; r[j + 2] = v.z; r[j + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < NP; ++j) r[j] = p[j];
  }
}
// `count` floats of each of `rows` global rows into shared rows of the padded layout
template <int NP, int PARTS>
__device__ __forceinline__ void stage_runs(float* dst, const float* src, size_t src_stride, int rows, int count, bool vec) {
  using L = RowLayout<NP, PARTS>;
  if (vec) {
    const int per = count >> 2;
    for (int i = threadIdx.x; i < rows * per; i += blockDim.x) {
      const int r = i / per, c = (i - r * per) << 2;
      cp_async16(dst + r * L::ROW + L::at(c), src + r * src_stride + c);
    }
  } else {
    for (int i = threadIdx.x; i < rows * count; i += blockDim.x) {
      const int r = i / count, c = i - r * count;
      cp_async4(dst + r * L::ROW + L::at(c), src + r * src_stride + c);
    }
  }
}

// a thread's NP state rows of one value column, from and to global memory: 16 bytes at a time where the state has
// exactly PARTS * NP rows (the threads of a column group then cover a column's `rows` values without a gap)
template <int NP, int PARTS> __device__ __forceinline__ void load_state(const float* st, int part, int rows, bool valid, float (&r)[NP]) {
  if (NP % 4 == 0 && rows == PARTS * NP) {
    if (valid) load_run<NP>(st + part * NP, r);
    else {
#pragma unroll
      for (int j = 0; j < NP; ++j) r[j] = 0.f;
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int n = part * NP + j;
    r[j] = (valid && n < rows) ? st[n] : 0.f;
  }
}
template <int NP, int PARTS> __device__ __forceinline__ void store_state(float* st, int part, int rows, const float (&r)[NP]) {
  if (NP % 4 == 0 && rows == PARTS * NP) {
#pragma unroll
    for (int j = 0; j < NP; j += 4) *reinterpret_cast<float4*>(st + part * NP + j) = make_float4(r[j], r[j + 1], r[j + 2], r[j + 3]);
    return;
  }
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int n = part * NP + j;
    if (n < rows) st[n] = r[j];
  }
}

template <int PARTS> __device__ __forceinline__ float group_sum(float v) {  // over PARTS neighbouring lanes
#pragma unroll
  for (int o = 1; o < PARTS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- selective state-space scan ----------------------------------------------------------------------
// xbc [tokens, inner + 2 groups * N] float32 (after the convolution): x | B | C;  dt_raw: column `head` of rows of
// `dt_stride` values (bfloat16 or float32);  y [tokens, inner] float32.
template <int NP, int VP, int PARTS>
__global__ void __launch_bounds__(SCAN_THREADS) selective_scan_kernel(const float* xbc, const void* dt_raw, int dt_is_bf16,
                                                             int dt_stride, const float* dt_bias, const float* a_log,
                                                             const float* d_skip, float* state, float* y,
                                                             const int* first_row, const int* slots, int heads, int vdim,
                                                             int n_state, int groups, int write_state, int n_slots,
                                                             int vec_bc, int vec_x) {
  constexpr int GROUPS = SCAN_THREADS / PARTS, NPAD = RowLayout<NP, PARTS>::ROW, RUN = RowLayout<NP, PARTS>::RUN, VB = GROUPS * VP;
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, part = tid % PARTS, grp = tid / PARTS;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  const int inner = heads * vdim, row_w = inner + 2 * groups * n_state;
  const int group = head / (heads / groups);
  constexpr int STAGE = CH * (2 * NPAD + VB);
  float* sdt = smem + 2 * STAGE;  // [CH]
  float* sdec = sdt + CH;         // [CH]
  const int cols = min(VB, vdim - v0);  // value columns this block really has
  if (n_state != PARTS * NP || cols != VB)
    for (int i = tid; i < 2 * STAGE; i += blockDim.x) smem[i] = 0.f;  // the padding stays zero from here on
  const double A = exp((double)a_log[head]);
  const float D = d_skip[head], bias = dt_bias[head];
  float s[VP][NP];
#pragma unroll
  for (int i = 0; i < VP; ++i) {
    const int v = v0 + grp * VP + i;
    load_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + (v < vdim ? v : 0)) * n_state, part, n_state, v < vdim, s[i]);
  }
  __syncthreads();
  auto issue = [&](int c0, int stage) {
    const int cn = min(CH, hi - c0);
    float* base = smem + stage * STAGE;
    const float* src = xbc + (size_t)c0 * row_w;
    stage_runs<NP, PARTS>(base, src + inner + (size_t)group * n_state, row_w, cn, n_state, vec_bc);
    stage_runs<NP, PARTS>(base + CH * NPAD, src + inner + (size_t)(groups + group) * n_state, row_w, cn, n_state, vec_bc);
    stage_rows(base + 2 * CH * NPAD, VB, src + (size_t)head * vdim + v0, row_w, cn, cols, vec_x);
    cp_async_commit();
  };
  if (lo < hi) issue(lo, 0);
  int stage = 0;
  for (int c0 = lo; c0 < hi; c0 += CH, stage ^= 1) {
    const int cn = min(CH, hi - c0);
    const bool more = c0 + CH < hi;
    if (more) issue(c0 + CH, stage ^ 1);
    if (tid < cn) {
      const size_t at = (size_t)(c0 + tid) * dt_stride + head;
      const float raw = dt_is_bf16 ? __bfloat162float(((const __nv_bfloat16*)dt_raw)[at]) : ((const float*)dt_raw)[at];
      // A decay is applied once a token and its error compounds over a sequence: the step size and the decay are taken
      // in double and rounded once (expf alone may be two units off in the last place)
      const double dt = softplus_d((double)raw + (double)bias);
      sdt[tid] = (float)dt;
      sdec[tid] = (float)exp(-A * dt);
    }
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const float* sB = smem + stage * STAGE;
    const float* sC = sB + CH * NPAD;
    const float* sx = sC + CH * NPAD;
    for (int t = 0; t < cn; ++t) {
      const float dec = sdec[t], dt = sdt[t];
      float xv[VP], dtx[VP], acc[VP];
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        xv[i] = sx[t * VB + grp * VP + i];
        dtx[i] = dt * xv[i];
        acc[i] = 0.f;
      }
      float b[NP], c[NP];
      load_run<NP>(sB + t * NPAD + part * RUN, b);
      load_run<NP>(sC + t * NPAD + part * RUN, c);
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float bj = b[j], cj = c[j];
#pragma unroll
        for (int i = 0; i < VP; ++i) {
          s[i][j] = fmaf(dec, s[i][j], dtx[i] * bj);
          acc[i] = fmaf(s[i][j], cj, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        acc[i] = group_sum<PARTS>(acc[i]);
        const int v = v0 + grp * VP + i;
        if (part == i && v < vdim) y[(size_t)(c0 + t) * inner + (size_t)head * vdim + v] = fmaf(D, xv[i], acc[i]);
      }
    }
    __syncthreads();  // this stage and sdt are free again
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < VP; ++i) {
      const int v = v0 + grp * VP + i;
      if (v >= vdim) continue;
      store_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + v) * n_state, part, n_state, s[i]);
    }
  }
}

// ---- gated delta rule --------------------------------------------------------------------------------
// What enters the recurrence, made ready for every token at once (a warp per token and head):
//   qkv [tokens, 2 kvheads * dim + heads * vdim] float32 (after the convolution): q | k | v;  q and k of every key head
//   become unit vectors in place, x / sqrt(sum(x^2) + 1e-6), q also times dim^-1/2
//   decay[t, h, n] = exp(-exp(a_log[h]) * softplus(a_raw[t, h, n] + dt_bias[h, n]));  beta[t, h] = sigmoid(beta_raw[t, h])
//   `per_head`: one decay a head, exp(-exp(a_log[h]) * softplus(a_raw[t, h] + dt_bias[h])), written to all its channels
//   a_raw is walked by its row stride `a_stride`
template <typename T>
__global__ void delta_prepare_kernel(float* qkv, const T* a_raw, int a_stride, int per_head, const T* beta_raw,
                                     int beta_stride, const float* dt_bias, const float* a_log, float* decay, float* beta,
                                     int heads, int kvheads, int dim, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int row_w = 2 * kvheads * dim + heads * vdim;
  const float q_scale = 1.f / sqrtf((float)dim);
  const int item = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);  // a warp per head
  if (item < 2 * kvheads + heads) {
    if (item < 2 * kvheads) {  // q heads, then k heads
      float* x = qkv + (size_t)t * row_w + (size_t)item * dim;
      float ss = 0.f;
      for (int n = lane; n < dim; n += 32) ss = fmaf(x[n], x[n], ss);
      const float inv = (item < kvheads ? q_scale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
      for (int n = lane; n < dim; n += 32) x[n] *= inv;
    } else {
      const int h = item - 2 * kvheads;
      const double A = exp((double)a_log[h]);  // decays compound over a sequence: taken in double, rounded once
      const size_t at = ((size_t)t * heads + h) * dim;
      if (per_head) {
        const float d = (float)exp(-A * softplus_d((double)to_f32(a_raw[(size_t)t * a_stride + h]) + (double)dt_bias[h]));
        for (int n = lane; n < dim; n += 32) decay[at + n] = d;
      } else {
        const T* ar = a_raw + (size_t)t * a_stride + (size_t)h * dim;
        for (int n = lane; n < dim; n += 32)
          decay[at + n] = (float)exp(-A * softplus_d((double)to_f32(ar[n]) + (double)dt_bias[(size_t)h * dim + n]));
      }
      if (lane == 0) beta[(size_t)t * heads + h] = sigmoid_f(to_f32(beta_raw[(size_t)t * beta_stride + h]));
    }
  }
}

// qkv as delta_prepare_kernel left it; decay [tokens, heads * dim], beta [tokens, heads]; o [tokens, heads * vdim]
template <int NP, int VP, int PARTS>
__global__ void __launch_bounds__(SCAN_THREADS) delta_rule_scan_kernel(const float* qkv, const float* decay, const float* beta,
                                                              float* state, float* o, const int* first_row,
                                                              const int* slots, int heads, int kvheads, int dim, int vdim,
                                                              int write_state, int n_slots, int vec_qk, int vec_g,
                                                              int vec_v) {
  constexpr int GROUPS = SCAN_THREADS / PARTS, NPAD = RowLayout<NP, PARTS>::ROW, RUN = RowLayout<NP, PARTS>::RUN, VB = GROUPS * VP;
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, part = tid % PARTS, grp = tid / PARTS;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  const int kvh = head / (heads / kvheads);
  const int row_w = 2 * kvheads * dim + heads * vdim;
  constexpr int STAGE = CH * (3 * NPAD + VB + 1);
  const int cols = min(VB, vdim - v0);
  if (dim != PARTS * NP || cols != VB)
    for (int i = tid; i < 2 * STAGE; i += blockDim.x) smem[i] = 0.f;  // the padding stays zero from here on
  float s[VP][NP];
#pragma unroll
  for (int i = 0; i < VP; ++i) {
    const int v = v0 + grp * VP + i;
    load_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + (v < vdim ? v : 0)) * dim, part, dim, v < vdim, s[i]);
  }
  __syncthreads();
  auto issue = [&](int c0, int stage) {
    const int cn = min(CH, hi - c0);
    float* base = smem + stage * STAGE;
    const float* src = qkv + (size_t)c0 * row_w;
    stage_runs<NP, PARTS>(base, src + (size_t)kvh * dim, row_w, cn, dim, vec_qk);
    stage_runs<NP, PARTS>(base + CH * NPAD, src + (size_t)(kvheads + kvh) * dim, row_w, cn, dim, vec_qk);
    stage_runs<NP, PARTS>(base + 2 * CH * NPAD, decay + ((size_t)c0 * heads + head) * dim, (size_t)heads * dim, cn, dim, vec_g);
    stage_rows(base + 3 * CH * NPAD, VB, src + 2 * (size_t)kvheads * dim + (size_t)head * vdim + v0, row_w, cn, cols, vec_v);
    stage_rows(base + 3 * CH * NPAD + CH * VB, 1, beta + (size_t)c0 * heads + head, heads, cn, 1, false);
    cp_async_commit();
  };
  if (lo < hi) issue(lo, 0);
  int stage = 0;
  for (int c0 = lo; c0 < hi; c0 += CH, stage ^= 1) {
    const int cn = min(CH, hi - c0);
    const bool more = c0 + CH < hi;
    if (more) issue(c0 + CH, stage ^ 1);
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const float* sq = smem + stage * STAGE;
    const float* sk = sq + CH * NPAD;
    const float* sg = sk + CH * NPAD;
    const float* sv = sg + CH * NPAD;
    const float* sbeta = sv + CH * VB;
    for (int t = 0; t < cn; ++t) {
      float q[NP], k[NP], g[NP];
      load_run<NP>(sk + t * NPAD + part * RUN, k);
      load_run<NP>(sg + t * NPAD + part * RUN, g);
      load_run<NP>(sq + t * NPAD + part * RUN, q);
      float acc[VP], u[VP];
#pragma unroll
      for (int i = 0; i < VP; ++i) acc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float gj = g[j], kj = k[j];
#pragma unroll
        for (int i = 0; i < VP; ++i) {
          s[i][j] *= gj;
          acc[i] = fmaf(s[i][j], kj, acc[i]);
        }
      }
      const float bt = sbeta[t];
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        u[i] = bt * (sv[t * VB + grp * VP + i] - group_sum<PARTS>(acc[i]));
        acc[i] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float kj = k[j], qj = q[j];
#pragma unroll
        for (int i = 0; i < VP; ++i) {
          s[i][j] = fmaf(kj, u[i], s[i][j]);
          acc[i] = fmaf(s[i][j], qj, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        acc[i] = group_sum<PARTS>(acc[i]);
        const int v = v0 + grp * VP + i;
        if (part == i && v < vdim) o[(size_t)(c0 + t) * heads * vdim + (size_t)head * vdim + v] = acc[i];
      }
    }
    __syncthreads();  // this stage is free again
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < VP; ++i) {
      const int v = v0 + grp * VP + i;
      if (v >= vdim) continue;
      store_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + v) * dim, part, dim, s[i]);
    }
  }
}

// ---- state matrices under scalar decays ---------------------------------------------------------------
// The first `cols` columns of the projection's rows, in float32: act 1 takes silu, and the first `q_cols` columns are
// multiplied by q_scale.  VEC values a thread.
template <typename T, int VEC>
__global__ void linear_prepare_kernel(const T* proj, int stride, float* out, int cols, int q_cols, float q_scale, int act,
                                      size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= total) return;
  const size_t t = i / cols;
  const int c = (int)(i - t * cols);
  float v[VEC];
  load_channels<VEC>(proj + t * stride + c, v);
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    if (act == 1) v[k] = v[k] * sigmoid_f(v[k]);
    if (c + k < q_cols) v[k] *= q_scale;
  }
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(out + i) = make_float4(v[0], v[1], v[2], v[3]);
  else out[i] = v[0];
}

// Exponential gates under a running maximum, a warp per (sequence, head).  gate_raw: column h of the rows is head h's
// input gate before its bias, column heads + h its forget gate; bias [2 heads] float32; cap > 0:
//   i = cap tanh((raw_i + bias_i) / cap);  f = logsigmoid(cap tanh((raw_f + bias_f) / cap))
//   m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m');  gates[t, h] = (a, b, exp(-m'))
// norm_state holds per slot and head the normalizer n (dim values) and then m, zeros for a new sequence.  m is left at
// its value after the step's last row; n as it was before the step is copied to norm_in [sequences, heads, dim], from
// where every block of the scan reads it (the scan's blocks do not all run at once, and one of them writes the new n
// into norm_state).  The lanes take a token each for the gates and exponentials; the maxima are walked in order.
template <typename T>
__global__ void exp_gates_kernel(const T* gate_raw, int stride, const float* bias, float cap, float* norm_state,
                                 float* norm_in, float* gates, const int* first_row, const int* slots, int heads, int dim,
                                 int write_state, int n_seqs, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= n_seqs * heads) return;
  const int seq = unit / heads, head = unit - seq * heads;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  float* st = norm_state + ((size_t)slot * heads + head) * (dim + 1);
  float m = st[dim];
  for (int e = lane; e < dim; e += 32) norm_in[(size_t)unit * dim + e] = st[e];
  const float bi = bias[head], bf = bias[heads + head];
  for (int base = lo; base < hi; base += 32) {
    const int t = base + lane;
    float gi = 0.f, gf = 0.f;
    if (t < hi) {
      gi = cap * tanhf((to_f32(gate_raw[(size_t)t * stride + head]) + bi) / cap);
      const float z = cap * tanhf((to_f32(gate_raw[(size_t)t * stride + heads + head]) + bf) / cap);
      gf = z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
    }
    float before = 0.f, after = 0.f;
    const int cn = min(32, hi - base);
#pragma unroll
    for (int j = 0; j < 32; ++j) {  // unrolled: the shuffles are issued ahead and only m waits for the step before
      const float ij = __shfl_sync(0xffffffffu, gi, j), fj = __shfl_sync(0xffffffffu, gf, j);
      const float next = j < cn ? fmaxf(fj + m, ij) : m;
      if (lane == j) {
        before = m;
        after = next;
      }
      m = next;
    }
    if (t < hi) {
      float* g = gates + ((size_t)t * heads + head) * 3;
      g[0] = expf(gf + before - after);
      g[1] = expf(gi - after);
      g[2] = expf(-after);
    }
  }
  if (write_state && lane == 0) st[dim] = m;
}

// qkv [tokens, 2 heads * dim + heads * vdim] float32: q | k | v, head by head; o [tokens, heads * vdim].
// GATED: per token and head (a, b, e) in gates [tokens, heads, 3]: S = a S + b k v^T, n = a n + b k,
// o = S^T q / (max(|n.q|, e) + 1e-6).  Every thread walks its rows of n beside its rows of the state columns (n is
// the state column of a value that is always one), so that a column group has n.q from the same shuffles as its sums
// and no thread waits for another group; n before the step comes from norm_in [sequences, heads, dim], and the first
// column group of a head's first block leaves the new n in norm_state [slots, heads, dim + 1].
// Else one decay a head (decay [heads]): S = decay S + k v^T, o = S^T q.
template <int NP, int VP, int PARTS, bool GATED>
__global__ void __launch_bounds__(SCAN_THREADS) decay_scan_kernel(const float* qkv, const float* gates, const float* decay,
                                                                  float* state, const float* norm_in, float* norm_state,
                                                                  float* o, const int* first_row, const int* slots,
                                                                  int heads, int dim, int vdim, int write_state,
                                                                  int n_slots, int vec_qk, int vec_v) {
  constexpr int GROUPS = SCAN_THREADS / PARTS, NPAD = RowLayout<NP, PARTS>::ROW, RUN = RowLayout<NP, PARTS>::RUN, VB = GROUPS * VP;
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, part = tid % PARTS, grp = tid / PARTS;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  const int row_w = 2 * heads * dim + heads * vdim;
  constexpr int STAGE = CH * (2 * NPAD + VB + 4);
  const int cols = min(VB, vdim - v0);
  if (dim != PARTS * NP || cols != VB)
    for (int i = tid; i < 2 * STAGE; i += blockDim.x) smem[i] = 0.f;  // the padding stays zero from here on
  float s[VP][NP];
#pragma unroll
  for (int i = 0; i < VP; ++i) {
    const int v = v0 + grp * VP + i;
    load_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + (v < vdim ? v : 0)) * dim, part, dim, v < vdim, s[i]);
  }
  float nn[GATED ? NP : 1];
  if constexpr (GATED) load_state<NP, PARTS>(norm_in + ((size_t)seq * heads + head) * dim, part, dim, true, nn);
  const float fixed = GATED ? 1.f : decay[head];
  __syncthreads();
  auto issue = [&](int c0, int stage) {
    const int cn = min(CH, hi - c0);
    float* base = smem + stage * STAGE;
    const float* src = qkv + (size_t)c0 * row_w;
    stage_runs<NP, PARTS>(base, src + (size_t)head * dim, row_w, cn, dim, vec_qk);
    stage_runs<NP, PARTS>(base + CH * NPAD, src + (size_t)(heads + head) * dim, row_w, cn, dim, vec_qk);
    stage_rows(base + 2 * CH * NPAD, VB, src + 2 * (size_t)heads * dim + (size_t)head * vdim + v0, row_w, cn, cols, vec_v);
    if (GATED) stage_rows(base + 2 * CH * NPAD + CH * VB, 4, gates + ((size_t)c0 * heads + head) * 3, (size_t)heads * 3, cn, 3, false);
    cp_async_commit();
  };
  if (lo < hi) issue(lo, 0);
  int stage = 0;
  for (int c0 = lo; c0 < hi; c0 += CH, stage ^= 1) {
    const int cn = min(CH, hi - c0);
    const bool more = c0 + CH < hi;
    if (more) issue(c0 + CH, stage ^ 1);
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const float* sq = smem + stage * STAGE;
    const float* sk = sq + CH * NPAD;
    const float* sv = sk + CH * NPAD;
    const float* sg = sv + CH * VB;
    // two tokens an iteration and two partial sums a column (even and odd rows): a token's loads and sums do not
    // wait for the token before it, only its state values do
#pragma unroll 2
    for (int t = 0; t < cn; ++t) {
      float q[NP], k[NP];
      load_run<NP>(sk + t * NPAD + part * RUN, k);
      load_run<NP>(sq + t * NPAD + part * RUN, q);
      const float a = GATED ? sg[t * 4] : fixed;
      const float b = GATED ? sg[t * 4 + 1] : 1.f;
      float acc[VP], odd[VP], val[VP], nq = 0.f, nq_odd = 0.f;
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        acc[i] = odd[i] = 0.f;
        val[i] = sv[t * VB + grp * VP + i] * b;
      }
#pragma unroll
      for (int j = 0; j < NP; j += 2) {
        const float k0 = k[j], q0 = q[j], k1 = k[j + 1], q1 = q[j + 1];
#pragma unroll
        for (int i = 0; i < VP; ++i) {
          s[i][j] = fmaf(a, s[i][j], k0 * val[i]);
          s[i][j + 1] = fmaf(a, s[i][j + 1], k1 * val[i]);
          acc[i] = fmaf(s[i][j], q0, acc[i]);
          odd[i] = fmaf(s[i][j + 1], q1, odd[i]);
        }
        if constexpr (GATED) {
          nn[j] = fmaf(a, nn[j], k0 * b);
          nn[j + 1] = fmaf(a, nn[j + 1], k1 * b);
          nq = fmaf(nn[j], q0, nq);
          nq_odd = fmaf(nn[j + 1], q1, nq_odd);
        }
      }
      float scale = 1.f;
      if constexpr (GATED) scale = 1.f / (fmaxf(fabsf(group_sum<PARTS>(nq + nq_odd)), sg[t * 4 + 2]) + 1e-6f);
#pragma unroll
      for (int i = 0; i < VP; ++i) {
        acc[i] = group_sum<PARTS>(acc[i] + odd[i]);
        const int v = v0 + grp * VP + i;
        if (part == i && v < vdim) o[(size_t)(c0 + t) * heads * vdim + (size_t)head * vdim + v] = acc[i] * scale;
      }
    }
    __syncthreads();  // this stage is free again
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < VP; ++i) {
      const int v = v0 + grp * VP + i;
      if (v >= vdim) continue;
      store_state<NP, PARTS>(state + (((size_t)slot * heads + head) * vdim + v) * dim, part, dim, s[i]);
    }
    if constexpr (GATED) {
      if (blockIdx.z == 0 && grp == 0) {
        float* st = norm_state + ((size_t)slot * heads + head) * (dim + 1);  // rows of dim + 1: no 16-byte stores
#pragma unroll
        for (int j = 0; j < NP; ++j)
          if (part * NP + j < dim) st[part * NP + j] = nn[j];
      }
    }
  }
}

// ---- norm over groups of a row, with a gate ----------------------------------------------------------
// x [tokens, width] float32; groups of `gs` values; weight[c % weight_period]; gate: columns of rows of gate_stride
// values.  gate_mode 1: x * silu(gate) before the norm;  2: sigmoid(gate) after the norm and the weight;  0: none.
// One warp per (token, group).
// four consecutive values at once (the pointer aligned to four values)
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const uint32_t*>(&a);
  t.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// TPU threads per (token, group): a warp, or a block of 256 where the groups are long; VEC values a thread at a time
// (4 where the sizes and addresses allow it)
template <typename T, int TPU, int VEC>
__global__ void gated_group_rmsnorm_kernel(const float* x, const T* gate, int gate_stride, int gate_mode,
                                           const float* weight, int weight_period, float eps, float factor, T* out,
                                           int n_tokens, int width, int gs) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x % TPU;
  const size_t unit = (size_t)blockIdx.x * (blockDim.x / TPU) + (threadIdx.x / TPU);
  const int per_row = width / gs;
  if (unit >= (size_t)n_tokens * per_row) return;  // TPU > 32: one unit a block, so the whole block alike
  const size_t t = unit / per_row;
  const int c0 = (int)(unit - t * per_row) * gs;
  const float* xr = x + t * width + c0;
  const T* gr = gate ? gate + t * gate_stride + c0 : nullptr;
  float ss = 0.f;
  for (int e = lane * VEC; e < gs; e += TPU * VEC) {
    float v[VEC], z[VEC];
    if constexpr (VEC == 4) {
      ld4(xr + e, v);
      if (gate_mode == 1) ld4(gr + e, z);
    } else {
      v[0] = xr[e];
      if (gate_mode == 1) z[0] = to_f32(gr[e]);
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if (gate_mode == 1) v[k] *= z[k] * sigmoid_f(z[k]);
      ss = fmaf(v[k], v[k], ss);
    }
  }
  float total;
  if constexpr (TPU == 32) total = warp_sum(ss);
  else total = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(total / (float)gs + eps);
  for (int e = lane * VEC; e < gs; e += TPU * VEC) {
    float v[VEC], z[VEC];
    if constexpr (VEC == 4) {
      ld4(xr + e, v);
      if (gate_mode != 0) ld4(gr + e, z);
    } else {
      v[0] = xr[e];
      if (gate_mode != 0) z[0] = to_f32(gr[e]);
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      if (gate_mode == 1) v[k] *= z[k] * sigmoid_f(z[k]);
      v[k] = v[k] * inv * weight[(c0 + e + k) % weight_period];
      if (gate_mode == 2) v[k] *= sigmoid_f(z[k]);
      if (gate_mode == 3) v[k] *= z[k] * sigmoid_f(z[k]);
      v[k] *= factor;
    }
    if constexpr (VEC == 4) st4(out + t * width + c0 + e, v);
    else out[t * width + c0 + e] = from_f32<T>(v[0]);
  }
}
}  // namespace

FMS_API int fms_scan_chunk_tokens() { return CH; }

FMS_API int fms_causal_conv(const void* x, int dtype, int stride, const float* w, const float* bias, float* tail,
                            const int* token_seq, const int* first_row, const int* slots, float* out, int n_tokens,
                            int n_seqs, int channels, int taps, int act, int write_state, int n_slots,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return fms_fail("causal_conv: %d taps (1..%d)", taps, MAX_TAPS);
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  const bool four = channels % 4 == 0 && stride % 4 == 0 && (uintptr_t)x % (4 * item) == 0 && (uintptr_t)out % 16 == 0;
  const int cpt = four ? 4 : 1;
  const dim3 grid((n_tokens + CONV_TOKENS - 1) / CONV_TOKENS, (channels / cpt + CONV_THREADS - 1) / CONV_THREADS);
#define FMS_CONV(CPT, TMAX)                                                                                          \
  fms_launch(causal_conv_kernel<T, CPT, TMAX>, grid, dim3(CONV_THREADS), 0, stream, (const T*)x, stride, w, bias,     \
             (const float*)tail, token_seq, first_row, slots, out, n_tokens, channels, taps, act, n_seqs, n_slots)
  FMS_DISPATCH_DTYPE(dtype, T, {
    if (four && taps <= 4) FMS_CONV(4, 4);
    else if (four) FMS_CONV(4, MAX_TAPS);
    else if (taps <= 4) FMS_CONV(1, 4);
    else FMS_CONV(1, MAX_TAPS);
    if (write_state && taps > 1)
      fms_launch(conv_tail_kernel<T>, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, stream, (const T*)x, stride, tail,
                 first_row, slots, channels, taps, n_seqs, n_slots);
  });
#undef FMS_CONV
  return fms_launch_status("causal_conv");
}

// How a scan is cut.  PARTS threads share a group of value columns and each holds NP of the state's rows: 8 threads
// by default; 16 or 32 where a model has so few heads and value columns that a single sequence would leave most
// multiprocessors idle (the choice looks at the model's sizes only, never at the batch, so a sequence's sums run in the
// same order whatever it is batched with).  VP value columns a thread: as many as still leave every multiprocessor
// four blocks, whose warps hide one another's latencies (the sums do not depend on it).
struct ScanShape {
  int parts, np, vp;
};
static ScanShape scan_shape(int n_seqs, int heads, int vdim, int rows, int few_default = 148) {
  ScanShape s;
  // FMS_B200_SCAN_FEW: blocks of a single sequence below which more threads share a column group (else the calling
  // scan's own number: 148, or more for a scan whose tokens cost little beside the wait for their sums)
  static int few_env = -2;
  if (few_env == -2) {
    const char* e = getenv("FMS_B200_SCAN_FEW");
    few_env = e ? atoi(e) : -1;
  }
  const int few = few_env >= 0 ? few_env : few_default;
  s.parts = 8;
  if ((long)heads * ((vdim + 15) / 16) < few && rows >= 64) s.parts = 16;
  if (s.parts == 16 && (long)heads * ((vdim + 7) / 8) < few && rows >= 128) s.parts = 32;
  const int need = (rows + s.parts - 1) / s.parts;
  s.np = need <= 2 ? 2 : (need <= 4 ? 4 : (need <= 8 ? 8 : (need <= 16 ? 16 : 32)));
  const int groups = SCAN_THREADS / s.parts;
  s.vp = 1;
  static int min_blocks = -1;  // FMS_B200_SCAN_BLOCKS: blocks that must remain for a thread to take more columns (592)
  if (min_blocks < 0) {
    const char* e = getenv("FMS_B200_SCAN_BLOCKS");
    min_blocks = e ? atoi(e) : 592;
  }
  for (int vp = s.np >= 32 ? 2 : 4; vp > 1; vp >>= 1)
    if ((long)n_seqs * heads * ((vdim + groups * vp - 1) / (groups * vp)) >= min_blocks && vdim >= groups * vp) {
      s.vp = vp;
      break;
    }
  return s;
}
static bool rows_allow_16(const void* base, long offset, long stride, int count) {
  return ((uintptr_t)base % 16 == 0) && offset % 4 == 0 && stride % 4 == 0 && count % 4 == 0;
}

#define FMS_SCAN_VP(LAUNCH, NP, PARTS)                                                  \
  do {                                                                                  \
    if (shape.vp == 4) LAUNCH(NP, 4, PARTS);                                             \
    else if (shape.vp == 2) LAUNCH(NP, 2, PARTS);                                        \
    else LAUNCH(NP, 1, PARTS);                                                           \
  } while (0)
#define FMS_SCAN_VP2(LAUNCH, NP, PARTS)                                                 \
  do {                                                                                  \
    if (shape.vp >= 2) LAUNCH(NP, 2, PARTS);                                             \
    else LAUNCH(NP, 1, PARTS);                                                           \
  } while (0)
#define FMS_SCAN_SHAPES(LAUNCH)                                                                        \
  do {                                                                                                 \
    if (shape.parts == 8) {                                                                            \
      if (shape.np == 2) FMS_SCAN_VP(LAUNCH, 2, 8); else if (shape.np == 4) FMS_SCAN_VP(LAUNCH, 4, 8);  \
      else if (shape.np == 8) FMS_SCAN_VP(LAUNCH, 8, 8); else if (shape.np == 16) FMS_SCAN_VP(LAUNCH, 16, 8); \
      else FMS_SCAN_VP2(LAUNCH, 32, 8);                                                                \
    } else if (shape.parts == 16) {                                                                    \
      if (shape.np <= 4) FMS_SCAN_VP(LAUNCH, 4, 16); else if (shape.np == 8) FMS_SCAN_VP(LAUNCH, 8, 16); \
      else FMS_SCAN_VP(LAUNCH, 16, 16);                                                                \
    } else {                                                                                           \
      if (shape.np <= 4) FMS_SCAN_VP(LAUNCH, 4, 32); else FMS_SCAN_VP(LAUNCH, 8, 32);                   \
    }                                                                                                  \
  } while (0)

FMS_API int fms_selective_scan(const float* xbc, const void* dt_raw, int dtype, int dt_stride, const float* dt_bias,
                               const float* a_log, const float* d_skip, float* state, float* y, const int* first_row,
                               const int* slots, int n_seqs, int heads, int vdim, int n_state, int groups,
                               int write_state, int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || n_state <= 0 || n_state > 256 || vdim <= 0)
    return fms_fail("selective_scan: %d heads, %d groups, state %d (up to 256), vdim %d", heads, groups, n_state, vdim);
  if (dtype != FMS_F32 && dtype != FMS_BF16) return fms_fail("selective_scan: dtype code %d", dtype);
  const ScanShape shape = scan_shape(n_seqs, heads, vdim, n_state);
  const int vb = SCAN_THREADS / shape.parts * shape.vp;  // value columns of a block
  const long row_w = (long)heads * vdim + 2L * groups * n_state;
  const int vec_bc = rows_allow_16(xbc, (long)heads * vdim, row_w, n_state) && n_state % 4 == 0 && shape.np % 4 == 0;
  const int vec_x = rows_allow_16(xbc, 0, row_w, vdim) && vb % 4 == 0 && vdim % vb == 0;
  const dim3 grid(n_seqs, heads, (vdim + vb - 1) / vb), block(SCAN_THREADS);
#define FMS_LAUNCH(NP, VP, PARTS)                                                                                       \
  do {                                                                                                                  \
    const size_t smem = ((size_t)2 * CH * (2 * RowLayout<NP, PARTS>::ROW + SCAN_THREADS / PARTS * VP) + 2 * CH) * sizeof(float); \
    cudaFuncSetAttribute(selective_scan_kernel<NP, VP, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    fms_launch(selective_scan_kernel<NP, VP, PARTS>, grid, block, smem, stream, xbc, dt_raw, dtype == FMS_BF16 ? 1 : 0, dt_stride, \
               dt_bias, a_log, d_skip, state, y, first_row, slots, heads, vdim, n_state, groups, write_state, n_slots,   \
               vec_bc, vec_x);                                                                                           \
  } while (0)
  FMS_SCAN_SHAPES(FMS_LAUNCH);
#undef FMS_LAUNCH
  return fms_launch_status("selective_scan");
}

// decay [tokens, heads * dim] and beta [tokens, heads]: float32 scratch of the caller's.  a_raw: rows of a_stride
// values, of which the first heads * dim (per_head: the first heads) are the decays' logits
FMS_API int fms_delta_rule_scan(float* qkv, const void* beta_raw, int dtype, int beta_stride, const void* a_raw,
                                int a_stride, int per_head, const float* dt_bias, const float* a_log, float* decay, float* beta, float* state, float* o,
                                const int* first_row, const int* slots, int n_tokens, int n_seqs, int heads, int kvheads,
                                int dim, int vdim, int write_state, int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (heads <= 0 || kvheads <= 0 || heads % kvheads || dim <= 0 || dim > 256 || vdim <= 0)
    return fms_fail("delta_rule_scan: %d heads over %d, dim %d (up to 256), vdim %d", heads, kvheads, dim, vdim);
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(delta_prepare_kernel<T>, dim3(n_tokens, (2 * kvheads + heads + 3) / 4), dim3(128), 0, stream, qkv, (const T*)a_raw,
                                          a_stride, per_head, (const T*)beta_raw, beta_stride, dt_bias, a_log, decay, beta, heads, kvheads, dim,
                                          vdim));
  const ScanShape shape = scan_shape(n_seqs, heads, vdim, dim);
  const int vb = SCAN_THREADS / shape.parts * shape.vp;  // value columns of a block
  const long row_w = 2L * kvheads * dim + (long)heads * vdim;
  const int vec_qk = rows_allow_16(qkv, 0, row_w, dim) && shape.np % 4 == 0;
  const int vec_g = rows_allow_16(decay, 0, (long)heads * dim, dim) && shape.np % 4 == 0;
  const int vec_v = rows_allow_16(qkv, 2L * kvheads * dim, row_w, vdim) && vdim % vb == 0 && vb % 4 == 0;
  const dim3 grid(n_seqs, heads, (vdim + vb - 1) / vb), block(SCAN_THREADS);
#define FMS_LAUNCH(NP, VP, PARTS)                                                                                       \
  do {                                                                                                                  \
    const size_t smem = ((size_t)2 * CH * (3 * RowLayout<NP, PARTS>::ROW + SCAN_THREADS / PARTS * VP + 1)) * sizeof(float); \
    cudaFuncSetAttribute(delta_rule_scan_kernel<NP, VP, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    fms_launch(delta_rule_scan_kernel<NP, VP, PARTS>, grid, block, smem, stream, (const float*)qkv, (const float*)decay, \
               (const float*)beta, state, o, first_row, slots, heads, kvheads, dim, vdim, write_state, n_slots, vec_qk,  \
               vec_g, vec_v);                                                                                            \
  } while (0)
  FMS_SCAN_SHAPES(FMS_LAUNCH);
#undef FMS_LAUNCH
  return fms_launch_status("delta_rule_scan");
}

// q | k | v of a step's rows in float32 from the first columns of the projection's rows (bfloat16 or float32):
// act 1 takes silu of every value; the first q_cols columns are multiplied by q_scale
FMS_API int fms_linear_prepare(const void* proj, int dtype, int stride, float* out, int n_tokens, int cols, int q_cols,
                               float q_scale, int act, cudaStream_t stream) {
  if (n_tokens <= 0 || cols <= 0) return 0;
  const size_t total = (size_t)n_tokens * cols;
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  const bool four = cols % 4 == 0 && stride % 4 == 0 && (uintptr_t)proj % (4 * item) == 0 && (uintptr_t)out % 16 == 0;
  if (four) {
    FMS_DISPATCH_DTYPE(dtype, T, fms_launch(linear_prepare_kernel<T, 4>, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0,
                                            stream, (const T*)proj, stride, out, cols, q_cols, q_scale, act, total));
  } else {
    FMS_DISPATCH_DTYPE(dtype, T, fms_launch(linear_prepare_kernel<T, 1>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                            stream, (const T*)proj, stride, out, cols, q_cols, q_scale, act, total));
  }
  return fms_launch_status("linear_prepare");
}

// qkv [tokens, 2 heads * dim + heads * vdim] float32.  With gate_raw (columns [i: heads | f: heads] of rows of
// gate_stride values, bias [2 heads], cap): exponential gates, with normalizer and running maximum in norm_state
// [slots, heads, dim + 1]; gates [tokens, heads, 3] and norm_in [sequences, heads, dim] are float32 scratch of the
// caller's.  Without: decay [heads].
FMS_API int fms_decay_scan(const float* qkv, const void* gate_raw, int dtype, int gate_stride, const float* gate_bias,
                           float cap, float* gates, float* norm_in, const float* decay, float* state, float* norm_state, float* o,
                           const int* first_row, const int* slots, int n_tokens, int n_seqs, int heads, int dim, int vdim,
                           int write_state, int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (heads <= 0 || dim <= 0 || dim > 256 || vdim <= 0)
    return fms_fail("decay_scan: %d heads, dim %d (up to 256), vdim %d", heads, dim, vdim);
  const bool gated = gate_raw != nullptr;
  if (gated && (!gate_bias || !gates || !norm_in || !norm_state || !(cap > 0.f))) return fms_fail("decay_scan: gates without bias, scratch, normalizer or cap");
  if (!gated && !decay) return fms_fail("decay_scan: neither gates nor decays");
  const long row_w = 2L * heads * dim + (long)heads * vdim;
  if (gated) {
    FMS_DISPATCH_DTYPE(dtype, T, fms_launch(exp_gates_kernel<T>, dim3((n_seqs * heads + 3) / 4), dim3(128), 0, stream,
                                            (const T*)gate_raw, gate_stride, gate_bias, cap, norm_state, norm_in, gates,
                                            first_row, slots, heads, dim, write_state, n_seqs, n_slots));
  }
  // under fixed decays a token is two multiply-adds a state value and one sum: 16 threads a column group (half the
  // rows a thread, twice the blocks) pay up to twice as many blocks as under gates (a prompt of 2,048 tokens, 32 heads
  // of 128 x 128: 4.5 ms against 5.8 for four layers; with gates 6.3 against 6.0)
  const ScanShape shape = scan_shape(n_seqs, heads, vdim, dim, gated ? 148 : 300);
  const int vb = SCAN_THREADS / shape.parts * shape.vp;  // value columns of a block
  const int vec_qk = rows_allow_16(qkv, 0, row_w, dim) && shape.np % 4 == 0;
  const int vec_v = rows_allow_16(qkv, 2L * heads * dim, row_w, vdim) && vdim % vb == 0 && vb % 4 == 0;
  const dim3 grid(n_seqs, heads, (vdim + vb - 1) / vb), block(SCAN_THREADS);
#define FMS_LAUNCH_G(NP, VP, PARTS, GATED)                                                                              \
  do {                                                                                                                  \
    const size_t smem = ((size_t)2 * CH * (2 * RowLayout<NP, PARTS>::ROW + SCAN_THREADS / PARTS * VP + 4)) * sizeof(float); \
    cudaFuncSetAttribute(decay_scan_kernel<NP, VP, PARTS, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    fms_launch(decay_scan_kernel<NP, VP, PARTS, GATED>, grid, block, smem, stream, qkv, (const float*)gates, decay, state, \
               (const float*)norm_in, norm_state, o, first_row, slots, heads, dim, vdim, write_state, n_slots, vec_qk, vec_v); \
  } while (0)
#define FMS_LAUNCH_T(NP, VP, PARTS) FMS_LAUNCH_G(NP, VP, PARTS, true)
#define FMS_LAUNCH_F(NP, VP, PARTS) FMS_LAUNCH_G(NP, VP, PARTS, false)
  if (gated) FMS_SCAN_SHAPES(FMS_LAUNCH_T);
  else FMS_SCAN_SHAPES(FMS_LAUNCH_F);
#undef FMS_LAUNCH_T
#undef FMS_LAUNCH_F
#undef FMS_LAUNCH_G
  return fms_launch_status("decay_scan");
}

FMS_API int fms_gated_group_rmsnorm(const float* x, const void* gate, int dtype, int gate_stride, int gate_mode,
                                    const float* weight, int weight_period, float eps, float factor, void* out,
                                    int n_tokens, int width, int group_size, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (group_size <= 0 || width % group_size || weight_period <= 0)
    return fms_fail("gated_group_rmsnorm: rows of %d in groups of %d", width, group_size);
  if (gate_mode != 0 && gate == nullptr) return fms_fail("gated_group_rmsnorm: a gate mode without a gate");
  const size_t units = (size_t)n_tokens * (width / group_size);
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  const bool four = group_size % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % (4 * item) == 0 &&
                    (gate == nullptr || (gate_stride % 4 == 0 && (uintptr_t)gate % (4 * item) == 0));
#define FMS_NORM(TPU, VEC, BLOCKS, THREADS)                                                                              \
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(gated_group_rmsnorm_kernel<T, TPU, VEC>, dim3((unsigned)(BLOCKS)), dim3(THREADS), 0,  \
                                          stream, x, (const T*)gate, gate_stride, gate_mode, weight, weight_period, eps, \
                                          factor, (T*)out, n_tokens, width, group_size))
  if (group_size >= 512) {
    if (four) FMS_NORM(256, 4, units, 256);
    else FMS_NORM(256, 1, units, 256);
  } else {
    if (four) FMS_NORM(32, 4, (units + 3) / 4, 128);
    else FMS_NORM(32, 1, (units + 3) / 4, 128);
  }
#undef FMS_NORM
  return fms_launch_status("gated_group_rmsnorm");
}
