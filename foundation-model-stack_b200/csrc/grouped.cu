// Products by groups of rows, and the routing of tokens to experts that makes such groups.
//
// grouped product: y[r, :] = x[r, :] . w[g]^T for the rows r of group g, w [groups, N, K].  The groups are either
//   ragged  — rows offsets[g] .. offsets[g + 1] - 1 of x and y (tokens sorted by expert; the offsets live on the device,
//             so a step needs no answer from the device before it launches), or
//   uniform — the same `rows` rows for every group, group g reading x at column g * x_group_offset and writing y at
//             column g * y_group_offset (the heads of one token matrix, each with a matrix of its own).
// With glu != 0, w[g] holds 2 N rows, [gate; up], and y = act(gate) * (up + 1) with gate cut off above `limit`, up
// clamped to +-limit and act(v) = v * sigmoid(alpha v): the gated unit of the routed experts.
// Sums are float32, each output element one chain over k in order, whatever else is in the launch.
//
// routing: scores = sigmoid(x . router^T) in float32; the `top` largest (the lower index among equals) are a token's
// experts and their scores its weights.  A (token, choice) pair becomes a row of the expert-sorted matrix:
// xs[row] = weight * x[token], rounded to the compute dtype.  After the experts, out[token] = the sum of its
// pairs' rows in the order of its choices, float32.
#include "common.cuh"


// Kernels of a step may start while the kernel before them is still running (programmatic dependent launch) and
// read what that kernel wrote right after griddepcontrol.wait.  No pointer here is declared __restrict__: the
// compiler must not turn such a read into a non-coherent load or move it ahead of the wait, and the few words of
// bookkeeping that the kernel before wrote (positions, offsets, groups) are read with ld_fresh (from L2).
#define __restrict__
__device__ __forceinline__ int ld_fresh(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcg(p); }

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// what an ungated product's sums go through: act 2 is the square of relu, anything else nothing
__device__ __forceinline__ float activated(float v, int act) {
  if (act == 2) {
    v = fmaxf(v, 0.f);
    v *= v;
  }
  return v;
}

__device__ __forceinline__ float glu_clamped(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f);
}

template <typename T, bool GLU>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           T* __restrict__ y, const int* __restrict__ offsets,
                                                           const int* __restrict__ tile_first, int groups, int rows,
                                                           int N, int K, long x_row_stride, long x_group_offset,
                                                           long y_row_stride, long y_group_offset, float limit,
                                                           float alpha, int act) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[GLU ? 2 : 1][BK][BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  int g, m0, m_end;
  if (offsets != nullptr) {
    const int tile = blockIdx.y;
    if (tile >= ld_fresh(tile_first + groups)) return;
    g = 0;
    while (g + 1 < groups && tile >= ld_fresh(tile_first + g + 1)) ++g;
    m0 = ld_fresh(offsets + g) + (tile - ld_fresh(tile_first + g)) * BM;
    m_end = ld_fresh(offsets + g + 1);
  } else {
    g = blockIdx.z;
    m0 = blockIdx.y * BM;
    m_end = rows;
    x += (size_t)g * x_group_offset;
    y += (size_t)g * y_group_offset;
  }
  const int n0 = blockIdx.x * BN;
  const T* wg = w + (size_t)g * (GLU ? 2 : 1) * N * K;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[GLU ? 2 : 1][TM][TN];
#pragma unroll
  for (int h = 0; h < (GLU ? 2 : 1); ++h)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[h][i][j] = 0.f;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
    float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[GLU ? 2 : 1][4];
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (gm < m_end && gk + i < K) xv[i] = to_f32(x[(size_t)gm * x_row_stride + gk + i]);
#pragma unroll
    for (int h = 0; h < (GLU ? 2 : 1); ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        wv[h][i] = (gn < N && gk + i < K) ? to_f32(wg[((size_t)h * N + gn) * K + gk + i]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xs[lk + i][lr] = xv[i];
#pragma unroll
      for (int h = 0; h < (GLU ? 2 : 1); ++h) ws[h][lk + i][lr] = wv[h][i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int h = 0; h < (GLU ? 2 : 1); ++h) {
        float b[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) b[j] = ws[h][k][tn + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[h][i][j] = fmaf(a[i], b[j], acc[h][i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= m_end) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      const float v = GLU ? glu_clamped(acc[0][i][j], acc[GLU ? 1 : 0][i][j], limit, alpha) : activated(acc[0][i][j], act);
      y[(size_t)gm * y_row_stride + gn] = from_f32<T>(v);
    }
  }
}

// Few rows a group (a decode step): a block per (group, 8 outputs), a warp per output (two with glu), its lanes striding
// over k; the warp walks the group's rows four at a time, so a group's matrix is read once however many of the step's
// rows it has (and not at all where it has none).  Ragged groups (offsets) or uniform ones (`rows` rows each, walked
// by strides as in the tiled kernel).  The sums are taken in another order than the tiles', so the two differ by
// rounding; a row's own sums do not depend on the other rows.
__device__ __forceinline__ void rows_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void rows_load8(const __nv_bfloat16* p, float* v) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __uint_as_float(u[k] << 16);
    v[2 * k + 1] = __uint_as_float(u[k] & 0xffff0000u);
  }
}

// pieces of a weight row that a lane of the row-walking kernel has in flight for an ungated product.  Measured through
// decode steps of 8 sequences over four layers with 16 experts of 3,584: one piece 2.00 ms, two 1.67, four 2.85 (the
// registers of four pieces and of their rows of x cost more blocks a multiprocessor than the loads in flight gain)
#ifndef FMS_ROW_PIECES
#define FMS_ROW_PIECES 2
#endif
// vec != 0: K, the strides and the group offsets are multiples of 8 values and the bases 16-byte aligned: a lane reads 8
// values at a time
template <typename T, bool GLU>
__global__ void __launch_bounds__(256) grouped_rows_kernel(const T* x, const T* w, T* y, const int* offsets, int groups,
                                                           int rows, int N, int K, long x_row_stride, long x_group_offset,
                                                           long y_row_stride, long y_group_offset, float limit,
                                                           float alpha, int vec, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  int r_lo = 0, r_hi = rows;
  if (offsets != nullptr) {
    r_lo = ld_fresh(offsets + g);
    r_hi = ld_fresh(offsets + g + 1);
  } else {
    x += (size_t)g * x_group_offset;
    y += (size_t)g * y_group_offset;
  }
  if (n >= N || r_lo >= r_hi) return;
  const T* w0 = w + ((size_t)g * (GLU ? 2 : 1) * N + n) * K;
  const T* w1 = w0 + (size_t)N * K;
  for (int r0 = r_lo; r0 < r_hi; r0 += 4) {
    const int nr = min(4, r_hi - r0);
    float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec && !GLU) {
      // PIECES pieces of the row a lane and iteration (k, k + 256, ...), all asked for before any is used: an ungated
      // product has one row a warp, and one piece of it in flight does not cover the memory's latency
      constexpr int PIECES = FMS_ROW_PIECES;
      float part[PIECES][4];
#pragma unroll
      for (int p = 0; p < PIECES; ++p) part[p][0] = part[p][1] = part[p][2] = part[p][3] = 0.f;
      for (int k = lane * 8; k < K; k += 256 * PIECES) {
        float wv[PIECES][8];
#pragma unroll
        for (int p = 0; p < PIECES; ++p)
          if (k + 256 * p < K) rows_load8(w0 + k + 256 * p, wv[p]);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < nr) {
#pragma unroll
            for (int p = 0; p < PIECES; ++p)
              if (k + 256 * p < K) {
                float xv[8];
                rows_load8(x + (size_t)(r0 + i) * x_row_stride + k + 256 * p, xv);
#pragma unroll
                for (int e = 0; e < 8; ++e) part[p][i] = fmaf(xv[e], wv[p][e], part[p][i]);
              }
          }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sum = part[0][i];
#pragma unroll
        for (int p = 1; p < PIECES; ++p) sum += part[p][i];
        a0[i] = sum;
      }
    } else if (vec) {
      for (int k = lane * 8; k < K; k += 256) {
        float wa[8], wb[8];
        rows_load8(w0 + k, wa);
        if (GLU) rows_load8(w1 + k, wb);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < nr) {
            float xv[8];
            rows_load8(x + (size_t)(r0 + i) * x_row_stride + k, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              a0[i] = fmaf(xv[e], wa[e], a0[i]);
              if (GLU) a1[i] = fmaf(xv[e], wb[e], a1[i]);
            }
          }
      }
    } else
    for (int k = lane; k < K; k += 32) {
      const float wa = to_f32(w0[k]), wb = GLU ? to_f32(w1[k]) : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < nr) {
          const float xv = to_f32(x[(size_t)(r0 + i) * x_row_stride + k]);
          a0[i] = fmaf(xv, wa, a0[i]);
          if (GLU) a1[i] = fmaf(xv, wb, a1[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < nr) {
        const float s0 = warp_sum(a0[i]), s1 = GLU ? warp_sum(a1[i]) : 0.f;
        if (lane == 0) y[(size_t)(r0 + i) * y_row_stride + n] = from_f32<T>(GLU ? glu_clamped(s0, s1, limit, alpha) : activated(s0, act));
      }
  }
}

// The gated unit alone, for rows [gate | up] that a library product left: out[r, f] = act(gate) * (up + 1), clamped
// as above.
template <typename T>
__global__ void gated_clamped_kernel(const T* gu, T* out, int hidden, float limit, float alpha, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / hidden;
    const int f = (int)(i - r * hidden);
    out[i] = from_f32<T>(glu_clamped(to_f32(gu[r * 2 * hidden + f]), to_f32(gu[r * 2 * hidden + hidden + f]), limit, alpha));
  }
}

__global__ void gated_clamped_vec_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out, int hidden, float limit, float alpha,
                                         int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = hidden >> 3;
  const long total = (long)n_rows * per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / per_row;
    const int f = (int)(i - r * per_row) * 8;
    float g[8], u[8];
    rows_load8(gu + r * 2 * hidden + f, g);
    rows_load8(gu + r * 2 * hidden + hidden + f, u);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 v = __floats2bfloat162_rn(glu_clamped(g[2 * k], u[2 * k], limit, alpha),
                                               glu_clamped(g[2 * k + 1], u[2 * k + 1], limit, alpha));
      o[k] = *reinterpret_cast<uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(out + r * hidden + f) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- routing -----------------------------------------------------------------------------------------
// One block per token.  logits in shared memory; warp 0 then takes the `top` largest one after the other.
constexpr int ROUTE_WARPS = 8;

template <typename T, typename TW>
__global__ void __launch_bounds__(32 * ROUTE_WARPS) route_kernel(const T* __restrict__ x, const TW* __restrict__ router,
                                                    int* __restrict__ expert, float* __restrict__ weight,
                                                    int dim, int experts, int top, int mode,
                                                    const float* __restrict__ correction, float route_scale) {
  extern __shared__ float sm[];  // dim values of x, then `experts` logits, then (mode 1) `experts` scores
  float* xs = sm;
  float* logit = sm + dim;
  float* score = logit + experts;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) xs[d] = to_f32(x[(size_t)t * dim + d]);
  __syncthreads();
  for (int e = warp; e < experts; e += ROUTE_WARPS) {
    const TW* wr = router + (size_t)e * dim;
    float a = 0.f, b = 0.f, c = 0.f, d4 = 0.f;  // four chains: the loads of one do not wait for another's sum
    int d = lane;
    for (; d + 96 < dim; d += 128) {
      a = fmaf(xs[d], to_f32(wr[d]), a);
      b = fmaf(xs[d + 32], to_f32(wr[d + 32]), b);
      c = fmaf(xs[d + 64], to_f32(wr[d + 64]), c);
      d4 = fmaf(xs[d + 96], to_f32(wr[d + 96]), d4);
    }
    for (; d < dim; d += 32) a = fmaf(xs[d], to_f32(wr[d]), a);
    a = warp_sum((a + b) + (c + d4));
    if (lane == 0) logit[e] = a;
  }
  __syncthreads();
  if (warp != 0) return;
  if (mode == 1) {
    // scores = softmax over all experts; the choice is by score + correction, the weights are the chosen scores over
    // their sum (+ 1e-20), times route_scale
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, logit[e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < experts; e += 32) den += expf(logit[e] - mx);
    den = warp_sum(den);
    for (int e = lane; e < experts; e += 32) {
      const float sc = expf(logit[e] - mx) / den;
      score[e] = sc;
      logit[e] = sc + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
  }
  float picked_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = logit[e];
      if (v > best || (v == best && e < at)) {
        best = v;
        at = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (at >= experts) at = k;  // every logit was NaN or -inf: any expert, so that nothing below reads outside
    if (lane == 0) {
      expert[(size_t)t * top + k] = at;
      weight[(size_t)t * top + k] = mode == 1 ? score[at] : 1.f / (1.f + expf(-best));
      logit[at] = -INFINITY;
    }
    if (mode == 1) picked_sum += score[at];
    __syncwarp();
  }
  if (mode == 1 && lane == 0) {
    const float f = route_scale / (picked_sum + 1e-20f);
    for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= f;
  }
}

// One block: counts every expert's pairs (in shared memory), then offsets [experts + 1], tile_first [experts + 1]
// (tiles of BM rows), and placed [experts] = 0: how many rows of each expert the next kernel has placed.
__global__ void __launch_bounds__(256) route_offsets_kernel(const int* __restrict__ expert, int n_pairs,
                                                            int* __restrict__ placed, int* __restrict__ offsets,
                                                            int* __restrict__ tile_first, int experts) {
  extern __shared__ int count[];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ld_fresh(expert + p);
    if (FMS_IN(e, experts)) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  int row = 0, tile = 0;
  for (int e = 0; e < experts; ++e) {
    const int c = count[e];
    offsets[e] = row;
    tile_first[e] = tile;
    row += c;
    tile += (c + BM - 1) / BM;
    placed[e] = 0;
  }
  offsets[experts] = row;
  tile_first[experts] = tile;
}

// One block per pair: takes the next free row of its expert and writes the weighted token there.
template <typename T>
__global__ void __launch_bounds__(128) route_scatter_kernel(const T* __restrict__ x, const int* __restrict__ expert,
                                                            const float* __restrict__ weight,
                                                            const int* __restrict__ offsets, int* __restrict__ placed,
                                                            int* __restrict__ row_of_pair, int* __restrict__ group_of_row,
                                                            T* __restrict__ xs, int dim, int top, int experts, int n_pairs,
                                                            int weighted) {
  __shared__ int where;
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x;
  const int e = ld_fresh(expert + p);
  if (!FMS_IN(e, experts)) return;
  if (threadIdx.x == 0) {
    where = ld_fresh(offsets + e) + atomicAdd(&placed[e], 1);
    row_of_pair[p] = where;
    if (FMS_IN(where, n_pairs)) group_of_row[where] = e;
  }
  __syncthreads();
  const int row = where;
  if (!FMS_IN(row, n_pairs)) return;
  const float wgt = weighted ? ld_fresh(weight + p) : 1.f;
  const T* src = x + (size_t)(p / top) * dim;
  T* dst = xs + (size_t)row * dim;
  if (weighted)
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = from_f32<T>(wgt * to_f32(src[d]));
  else
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = src[d];
}

template <typename T>
__global__ void __launch_bounds__(256) route_gather_kernel(const T* __restrict__ ys, const int* __restrict__ row_of_pair,
                                                           T* __restrict__ out, int dim, int top, int n_pairs,
                                                           const float* weight) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int rows_of_token[];  // then, as floats, the pairs' weights
  float* weight_of_token = reinterpret_cast<float*>(rows_of_token + top);
  const int t = blockIdx.x;
  for (int k = threadIdx.x; k < top; k += blockDim.x) {
    rows_of_token[k] = ld_fresh(row_of_pair + (size_t)t * top + k);
    weight_of_token[k] = weight ? ld_fresh(weight + (size_t)t * top + k) : 1.f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = rows_of_token[k];
      if (FMS_IN(row, n_pairs)) a = fmaf(weight_of_token[k], to_f32(ys[(size_t)row * dim + d]), a);
    }
    out[(size_t)t * dim + d] = from_f32<T>(a);
  }
}
}  // namespace

FMS_API int fms_grouped_tile_rows() { return BM; }

// offsets null: uniform groups of `rows` rows; else ragged groups, `rows` = all rows of x, and tile_first as
// fms_route leaves it.  few_rows != 0: the kernel that walks each group's rows (a decode step).
// glu: 0 plain, 1 the gated unit over [gate; up] rows, 2 an ungated product whose sums are squared where positive.
FMS_API int fms_grouped_linear(const void* x, const void* w, void* y, int dtype, const int* offsets, const int* tile_first,
                               const int* group_of_row, int groups, int rows, int N, int K, long x_row_stride,
                               long x_group_offset, long y_row_stride, long y_group_offset, int glu, float limit,
                               float alpha, int few_rows, cudaStream_t stream) {
  if (rows <= 0 || groups <= 0 || N <= 0) return 0;
  if (K <= 0) return fms_fail("grouped_linear: K %d", K);
  const int act = glu == 2 ? 2 : 0;
  glu = glu == 1 ? 1 : 0;
  if (few_rows) {
    if (groups > 65535) return fms_fail("grouped_linear: %d groups are more than the row-by-row kernel takes", groups);
    dim3 grid((N + 7) / 8, groups);
    const int vec = K % 8 == 0 && x_row_stride % 8 == 0 && x_group_offset % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
                    ((uintptr_t)w & 15) == 0;
    FMS_DISPATCH_DTYPE(dtype, T, {
      if (glu)
        fms_launch(grouped_rows_kernel<T, true>, grid, dim3(256), 0, stream, (const T*)x, (const T*)w, (T*)y, offsets, groups,
                   rows, N, K, x_row_stride, x_group_offset, y_row_stride, y_group_offset, limit, alpha, vec, act);
      else
        fms_launch(grouped_rows_kernel<T, false>, grid, dim3(256), 0, stream, (const T*)x, (const T*)w, (T*)y, offsets, groups,
                   rows, N, K, x_row_stride, x_group_offset, y_row_stride, y_group_offset, limit, alpha, vec, act);
    });
    return fms_launch_status("grouped_linear (few rows)");
  }
  dim3 grid((N + BN - 1) / BN, 1, 1);
  if (offsets != nullptr) {
    if (tile_first == nullptr) return fms_fail("grouped_linear: ragged groups need tile_first");
    grid.y = (rows + BM - 1) / BM + groups;
  } else {
    grid.y = (rows + BM - 1) / BM;
    grid.z = groups;
  }
  if (grid.y > 65535 || grid.z > 65535) return fms_fail("grouped_linear: %d rows, %d groups are more than one launch takes", rows, groups);
  FMS_DISPATCH_DTYPE(dtype, T, {
    if (glu)
      fms_launch(grouped_gemm_kernel<T, true>, grid, dim3(256), 0, stream, (const T*)x, (const T*)w, (T*)y, offsets,
                 tile_first, groups, rows, N, K, x_row_stride, x_group_offset, y_row_stride, y_group_offset, limit, alpha, act);
    else
      fms_launch(grouped_gemm_kernel<T, false>, grid, dim3(256), 0, stream, (const T*)x, (const T*)w, (T*)y, offsets,
                 tile_first, groups, rows, N, K, x_row_stride, x_group_offset, y_row_stride, y_group_offset, limit, alpha, act);
  });
  return fms_launch_status("grouped_linear");
}

// x [n_tokens, dim] in `dtype`, router [experts, dim] in `router_dtype`.  Out: expert, weight [n_tokens, top];
// offsets, tile_first [experts + 1]; row_of_pair [n_tokens * top]; group_of_row [n_tokens * top]; xs [n_tokens * top, dim].
// counts [experts] is scratch: the rows of each expert that are placed so far.
// mode 0: scores sigmoid(logit), the rows of xs are the tokens' times their weights.  mode 1: scores softmax(logits), the
// choice by score + correction [experts] (float32 or null), weights the chosen scores over their sum times route_scale;
// the rows of xs are the tokens' as they are and fms_route_gather takes the weights.
FMS_API int fms_route(const void* x, int dtype, const void* router, int router_dtype, int* expert, float* weight, int* counts,
                      int* offsets, int* tile_first, int* row_of_pair, int* group_of_row, void* xs, int n_tokens, int dim,
                      int experts, int top, int mode, const float* correction, float route_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || experts <= 0 || top <= 0 || top > experts) return fms_fail("route: dim %d, experts %d, top %d", dim, experts, top);
  if (mode != 0 && mode != 1) return fms_fail("route: mode %d", mode);
  const size_t smem = ((size_t)dim + 2 * (size_t)experts) * sizeof(float);
  if (smem > 200 * 1024) return fms_fail("route: rows of %d values and %d experts do not fit shared memory", dim, experts);
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(router_dtype, TW, {
    if (smem > 48 * 1024) cudaFuncSetAttribute(route_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    fms_launch(route_kernel<T, TW>, dim3(n_tokens), dim3(32 * ROUTE_WARPS), smem, stream, (const T*)x, (const TW*)router, expert, weight,
               dim, experts, top, mode, correction, route_scale);
  }));
  if (fms_launch_status("route")) return 1;
  const int n_pairs = n_tokens * top;
  fms_launch(route_offsets_kernel, dim3(1), dim3(256), sizeof(int) * experts, stream, (const int*)expert, n_pairs, counts,
             offsets, tile_first, experts);
  if (fms_launch_status("route (offsets)")) return 1;
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(route_scatter_kernel<T>, dim3(n_pairs), dim3(128), 0, stream, (const T*)x, (const int*)expert,
                                (const float*)weight, (const int*)offsets, counts, row_of_pair, group_of_row, (T*)xs, dim,
                                top, experts, n_pairs, mode == 0 ? 1 : 0));
  return fms_launch_status("route (scatter)");
}

// y = relu(y)^2 in place: the activation of ungated experts after a library product
template <typename T>
__global__ void relu_squared_kernel(T* y, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    y[i] = from_f32<T>(activated(to_f32(y[i]), 2));
}

__global__ void relu_squared_vec_kernel(__nv_bfloat16* y, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8];
    rows_load8(y + 8 * i, v);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 b = __floats2bfloat162_rn(activated(v[2 * k], 2), activated(v[2 * k + 1], 2));
      o[k] = *reinterpret_cast<uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(y + 8 * i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

FMS_API int fms_relu_squared(void* y, int dtype, long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (dtype == FMS_BF16 && total % 8 == 0 && ((uintptr_t)y & 15) == 0) {
    const long total8 = total / 8;
    const int blocks = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
    fms_launch(relu_squared_vec_kernel, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)y, (size_t)total8);
    return fms_launch_status("relu_squared");
  }
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(relu_squared_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)y, (size_t)total));
  return fms_launch_status("relu_squared");
}

FMS_API int fms_gated_clamped(const void* gu, void* out, int dtype, int n_rows, int hidden, float limit, float alpha,
                              cudaStream_t stream) {
  if (n_rows <= 0 || hidden <= 0) return 0;
  if (dtype == FMS_BF16 && hidden % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const long total8 = (long)n_rows * (hidden / 8);
    const int blocks8 = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
    fms_launch(gated_clamped_vec_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
               hidden, limit, alpha, n_rows);
    return fms_launch_status("gated_clamped");
  }
  const size_t total = (size_t)n_rows * hidden;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(gated_clamped_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)gu, (T*)out, hidden,
                                limit, alpha, total));
  return fms_launch_status("gated_clamped");
}

// weight: [n_tokens, top] float32 that multiply the pairs' rows, or null for their plain sum
FMS_API int fms_route_gather(const void* ys, int dtype, const int* row_of_pair, void* out, int n_tokens, int dim, int top,
                             const float* weight, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(route_gather_kernel<T>, dim3(n_tokens), dim3(256), 2 * sizeof(int) * top, stream, (const T*)ys, row_of_pair,
                                (T*)out, dim, top, n_tokens * top, weight));
  return fms_launch_status("route_gather");
}
