// Attention over a cache of latent rows: every cached position holds ONE row [c | kr] for all heads — c (`rank`
// values) is the normed down-projection from which a head's keys and values would be made by two matrices, kr (`rot`
// values) the rotated key part that all heads share.  The head's up-projections are folded into the query and taken
// out of the result, so nothing but the latent rows is ever read:
//   score_h(i, j) = (ql_h(i) . c(j) + qr_h(i) . kr(j)) * scale        ql_h = W_uk,h^T q_h (made before this kernel)
//   p = softmax over j <= i, with one more term exp(sink_h) in the denominator that has no key and no value
//   ol_h(i) = sum_j p(i, j) c(j), times sigmoid(gate_h(i))             the head's value is W_uv,h ol_h (made after)
// Scores, softmax and sums are float32.  The cache is the block cache of the other attention kernels with one
// key head of rank + rot values and no value plane.
//
// latent_prepare (c and kr may also come from a matrix of their own, `kv`; pairs by halves and a constant on the sines
// and cosines are options): from the fused projection [q heads (dim + rot each) | c (rank) | kr (rot) | gates (heads)] of a
// step's rows it norms c (RMS, a gain per value), rotates kr and every head's rot part by the row's position
// (adjacent pairs (2i, 2i+1), the first rot_dims values, angle = position * inv_freq[i], float32), writes [c | kr]
// into the cache at the row's slot and place and the rotated query parts into q_full[:, h, rank:].
#include "common.cuh"


// Kernels of a step may start while the kernel before them is still running (programmatic dependent launch) and
// read what that kernel wrote right after griddepcontrol.wait.  No pointer here is declared __restrict__: the
// compiler must not turn such a read into a non-coherent load or move it ahead of the wait, and the few words of
// bookkeeping that the kernel before wrote (positions, offsets, groups) are read with ld_fresh (from L2).
#define __restrict__
__device__ __forceinline__ int ld_fresh(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcg(p); }

namespace {
constexpr int SPLIT = 256;  // keys of one split of a decode step: fixed, so a sequence's sums depend on its length only
constexpr int KT = 32;      // keys brought into shared memory at a time
constexpr int HG = 8;       // heads a block takes
constexpr int THREADS = 256;

// Value j (< 2 half) of a rotated run: pairs (2i, 2i + 1), or with `halves` (i, i + half), turned by position * inv_freq[i];
// rot_mult multiplies sine and cosine (1 for a plain rotation).
template <typename T>
__device__ __forceinline__ float rotated(const T* src, int j, int half, int halves, float position, const float* inv_freq,
                                         float rot_mult) {
  const int pair = halves ? (j < half ? j : j - half) : j >> 1;
  const bool second = halves ? j >= half : (j & 1);
  float sn, cs;
  sincosf(position * inv_freq[pair], &sn, &cs);
  sn *= rot_mult;
  cs *= rot_mult;
  const float a = to_f32(src[halves ? pair : 2 * pair]), b = to_f32(src[halves ? pair + half : 2 * pair + 1]);
  return second ? b * cs + a * sn : a * cs - b * sn;
}

template <typename T, typename TG>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const T* __restrict__ proj, int proj_width, T* __restrict__ q_full, const TG* __restrict__ c_gain, float eps,
    const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
    const int* __restrict__ position_ids, const int* __restrict__ token_seq, const int* __restrict__ slots,
    T* __restrict__ cache, const int* __restrict__ table, int table_stride, int block_tokens, int heads, int dim, int rot,
    int rank, int write_cache, int n_seqs, int n_slots, int n_blocks, int* __restrict__ error_flag, int halves,
    float rot_mult, const T* __restrict__ kv, int kv_width) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * proj_width;
  const int q_cols = heads * (dim + rot);
  const float position = (float)(position_ids ? ld_fresh(position_ids + t) : ld_fresh(positions + t));
  const int width = rank + rot;
  // the rotated part of every head's query
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
    const int h = i / rot, j = i - h * rot;
    const T* src = row + (size_t)h * (dim + rot) + dim;
    float v;
    if (j < 2 * half) {
      v = rotated(src, j, half, halves, position, inv_freq, rot_mult);
    } else {
      v = to_f32(src[j]);
    }
    q_full[((size_t)t * heads + h) * width + rank + j] = from_f32<T>(v);
  }
  if (!write_cache) return;
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, n_slots)) return;
  const int pos = ld_fresh(positions + t);
  const int blk = table[(size_t)slot * table_stride + pos / block_tokens];
  if (blk < 0 || blk >= n_blocks) {
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  T* dst = cache + ((size_t)blk * block_tokens + pos % block_tokens) * width;
  // [c | kr] follow the queries in the row, or are the first columns of a matrix of their own (queries that come from
  // another projection)
  const T* c = kv ? kv + (size_t)t * kv_width : row + q_cols;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_f32(c[d]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_f32<T>(to_f32(c[d]) * inv * to_f32(c_gain[d]));
  const T* kr = c + rank;
  for (int j = threadIdx.x; j < rot; j += blockDim.x) {
    float v;
    if (j < 2 * half) {
      v = rotated(kr, j, half, halves, position, inv_freq, rot_mult);
    } else {
      v = to_f32(kr[j]);
    }
    dst[rank + j] = from_f32<T>(v);
  }
}

// A run of columns of a wider matrix, normed row by row: out[t, :n] = x[t, off : off + n] / sqrt(mean(.^2) + eps) * gain
// (queries that go through a latent of their own).  A block a row; with `vec` (n and the row stride multiples of 4
// values, the bases aligned to four values) a thread takes four values at a time; float32 arithmetic.
template <typename T> __device__ __forceinline__ void qn_load4(const T* p, float* v);
template <> __device__ __forceinline__ void qn_load4<float>(const float* p, float* v) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void qn_load4<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}

template <typename T, typename TG>
__global__ void __launch_bounds__(128) latent_query_norm_kernel(const T* x, int stride, int n, const TG* gain, float eps,
                                                               T* out, int n_tokens, int vec) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = x + (size_t)t * stride;
  float ss = 0.f;
  if (vec) {
    for (int d = threadIdx.x * 4; d < n; d += blockDim.x * 4) {
      float v[4];
      qn_load4<T>(row + d, v);
      ss += (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
    }
  } else {
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
      const float v = to_f32(row[d]);
      ss += v * v;
    }
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  if (vec) {
    for (int d = threadIdx.x * 4; d < n; d += blockDim.x * 4) {
      float v[4];
      qn_load4<T>(row + d, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) out[(size_t)t * n + d + e] = from_f32<T>(v[e] * inv * to_f32(gain[d + e]));
    }
  } else {
    for (int d = threadIdx.x; d < n; d += blockDim.x) out[(size_t)t * n + d] = from_f32<T>(to_f32(row[d]) * inv * to_f32(gain[d]));
  }
}

struct LatentArgs {
  const void* q;      // [tokens, heads, rank + rot]
  void* out;          // [tokens, heads, rank]
  const void* cache;  // [blocks, block_tokens, rank + rot]
  const void* gate;   // first gate logit of row 0: gate[t * gate_stride + h]; null: no gate
  const void* sink;   // [heads] or null
  const int* table;
  const int* slots;
  const int* token_seq;
  const int* positions;
  float* part_o;   // [tokens, heads, splits, rank]
  float* part_ml;  // [tokens, heads, splits, 2]
  long gate_stride;
  int table_stride, block_tokens, heads, rank, rot, n_splits, n_seqs, n_slots, n_blocks;
  float scale;
  int window;  // > 0: the row at position p sees the keys p - window + 1 .. p only
};

// One block per (row, split of keys, group of HG heads).  Keys come KT at a time into shared memory as float32; a warp
// takes the scores of one head (a lane a key), then 32 threads a head take the sums over the keys for rank / 32
// values each (NACC of them in registers).
template <typename T, typename TS, int NACC>
__global__ void __launch_bounds__(THREADS) latent_attention_kernel(LatentArgs a) {
  extern __shared__ float sm[];
  const int width = a.rank + a.rot;
  const int kstride = width | 1;  // odd: lanes that read the same value of different keys meet different banks
  float* qs = sm;                      // [HG][width]
  float* ks = qs + HG * width;         // [KT][kstride]
  float* ps = ks + KT * kstride;       // [HG][KT]
  float* alpha = ps + HG * KT;         // [HG]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * HG;
  const int nh = min(HG, a.heads - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = ld_fresh(a.positions + t);
  const int seq = a.token_seq[t];
  if (!FMS_IN(seq, a.n_seqs)) return;
  const int slot = a.slots[seq];
  if (!FMS_IN(slot, a.n_slots)) return;
  const bool whole = a.n_splits == 1;  // one split takes all keys and writes the result itself
  const int seen = a.window > 0 ? max(0, pos - a.window + 1) : 0;  // the first key this row sees
  const int hi = whole ? pos + 1 : min(pos + 1, split * SPLIT + SPLIT);
  if (hi <= seen) return;  // a split before the window: the merge does not look at it
  const int lo = max(whole ? 0 : split * SPLIT, seen / KT * KT);  // tiles stay aligned; keys before `seen` are masked
  const T* q = (const T*)a.q + ((size_t)t * a.heads + h0) * width;
  for (int i = threadIdx.x; i < nh * width; i += THREADS) qs[i] = to_f32(q[i]);
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;  // of head `warp`, kept alike by all lanes of the warp
  const T* cache = (const T*)a.cache;
  for (int k0 = lo; k0 < hi; k0 += KT) {
    __syncthreads();  // the last tile's sums are taken (and, the first time, q is in place)
    const int nk = min(KT, hi - k0);
    {
      // a tile of KT keys lies inside one cache block (KT divides the block's tokens): one look at the table; a warp
      // brings whole rows, its lanes striding over a row
      const int blk = a.table[(size_t)slot * a.table_stride + k0 / a.block_tokens];
      const bool held = blk >= 0 && blk < a.n_blocks;
      const T* src = cache + ((size_t)(held ? blk : 0) * a.block_tokens + k0 % a.block_tokens) * width;
      for (int j = warp; j < nk; j += THREADS / 32)
        for (int d = lane; d < width; d += 32) ks[j * kstride + d] = held ? to_f32(src[(size_t)j * width + d]) : 0.f;
    }
    __syncthreads();
    if (warp < nh) {
      float s = -INFINITY;
      const bool counts = lane < nk && k0 + lane >= seen;
      if (counts) {
        const float* qh = qs + warp * width;
        const float* kj = ks + lane * kstride;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;  // four chains: none waits for the one before
        int d = 0;
        for (; d + 3 < width; d += 4) {
          d0 = fmaf(qh[d], kj[d], d0);
          d1 = fmaf(qh[d + 1], kj[d + 1], d1);
          d2 = fmaf(qh[d + 2], kj[d + 2], d2);
          d3 = fmaf(qh[d + 3], kj[d + 3], d3);
        }
        for (; d < width; ++d) d0 = fmaf(qh[d], kj[d], d0);
        s = ((d0 + d1) + (d2 + d3)) * a.scale;
      }
      const float m_new = fmaxf(m_run, warp_max(s));
      const float p = counts ? expf(s - m_new) : 0.f;
      const float al = m_run == -INFINITY ? 0.f : expf(m_run - m_new);  // 0 the first time
      l_run = l_run * al + warp_sum(p);
      m_run = m_new;
      ps[warp * KT + lane] = p;
      if (lane == 0) alpha[warp] = al;
    }
    __syncthreads();
    {
      const int h = threadIdx.x >> 5;  // 32 threads a head
      if (h < nh) {
        const float al = alpha[h];
        const float* ph = ps + h * KT;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= al;
        for (int j = 0; j < nk; ++j) {
          const float pj = ph[j];
          const float* cj = ks + j * kstride + lane;
#pragma unroll
          for (int i = 0; i < NACC; ++i)
            if (lane + 32 * i < a.rank) acc[i] = fmaf(pj, cj[32 * i], acc[i]);
        }
      }
    }
  }
  if (warp >= nh) return;
  const int h = h0 + warp;
  if (whole) {
    float m = m_run, denom = l_run;
    if (a.sink) {
      const float sk = to_f32(((const TS*)a.sink)[h]);
      m = fmaxf(m_run, sk);
      denom = l_run * expf(m_run - m) + expf(sk - m);
    }
    float f = expf(m_run - m) / denom;
    if (a.gate) f *= 1.f / (1.f + expf(-to_f32(((const T*)a.gate)[(size_t)t * a.gate_stride + h])));
    T* o = (T*)a.out + ((size_t)t * a.heads + h) * a.rank;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < a.rank) o[d] = from_f32<T>(acc[i] * f);
    }
  } else {
    const size_t at = ((size_t)t * a.heads + h) * a.n_splits + split;
    if (lane == 0) {
      a.part_ml[2 * at] = m_run;
      a.part_ml[2 * at + 1] = l_run;
    }
    float* o = a.part_o + at * a.rank;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < a.rank) o[d] = acc[i];
    }
  }
}

// Merges a row's splits: a block per (row, head).
template <typename T, typename TS>
__global__ void __launch_bounds__(128) latent_combine_kernel(LatentArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = ld_fresh(a.positions + t);
  const int used = min(a.n_splits, pos / SPLIT + 1);
  const int s_lo = a.window > 0 ? min(max(0, pos - a.window + 1) / SPLIT, used - 1) : 0;  // splits before the window hold nothing
  const size_t at = ((size_t)t * a.heads + h) * a.n_splits;
  float m = a.sink ? to_f32(((const TS*)a.sink)[h]) : -INFINITY;
  for (int s = s_lo; s < used; ++s) m = fmaxf(m, a.part_ml[2 * (at + s)]);
  float denom = a.sink ? expf(to_f32(((const TS*)a.sink)[h]) - m) : 0.f;
  for (int s = s_lo; s < used; ++s) denom += a.part_ml[2 * (at + s) + 1] * expf(a.part_ml[2 * (at + s)] - m);
  float f = 1.f / denom;
  if (a.gate) f *= 1.f / (1.f + expf(-to_f32(((const T*)a.gate)[(size_t)t * a.gate_stride + h])));
  T* o = (T*)a.out + ((size_t)t * a.heads + h) * a.rank;
  for (int d = threadIdx.x; d < a.rank; d += blockDim.x) {
    float v = 0.f;
    for (int s = s_lo; s < used; ++s) v = fmaf(a.part_o[(at + s) * a.rank + d], expf(a.part_ml[2 * (at + s)] - m), v);
    o[d] = from_f32<T>(v * f);
  }
}

// ---- many rows, bfloat16: the two products on the tensor cores (mma.sync m16n8k16, float32 sums) ---------------
// A block owns MR = 32 rows: `tq` consecutive tokens of one sequence times `hb` heads (tq * hb = 32), all of which
// read the same keys.  Keys come MK = 32 at a time into shared memory (cp.async, two stages; keys beyond the
// tile's last position are zeros).  Per tile: (A) warp w takes the scores of 16 rows against 8 keys over the whole
// row width; (B) eight threads a row take the running maximum, the probabilities (bfloat16, as in every
// flash-attention kernel) and the sum; (C) warp w adds P . c for 16 rows and a quarter of the latent's columns
// (rank / 4, its share of the accumulator in registers), c being read as it lies in the key tile.
// With n_splits > 1 (a decode step: tq = 1, the block's rows are one token's heads) block z takes the keys of split z
// (SPLIT keys) and leaves its unnormed sums, maximum and sum for latent_combine_kernel.
constexpr int MR = 32, MK = 32;

__device__ __forceinline__ void lat_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lat_ldmatrix(uint32_t* r, const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(row)));
}
__device__ __forceinline__ void lat_ldmatrix_trans(uint32_t* r, const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(row)));
}
__device__ __forceinline__ void lat_copy16(void* smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes) : "memory");
}

template <typename TS, int NT>
__global__ void __launch_bounds__(256) latent_prefill_mma_kernel(LatentArgs a, const int* tiles, const int* first_row,
                                                                 int tq, int hb) {
  extern __shared__ __align__(16) unsigned char lat_smem[];
  const int width = a.rank + a.rot;
  const int rowb = width * 2 + 16, prowb = MK * 2 + 16;
  unsigned char* qs = lat_smem;
  unsigned char* ks = qs + MR * rowb;
  float* ss = reinterpret_cast<float*>(ks + 2 * MK * rowb);
  unsigned char* ps = reinterpret_cast<unsigned char*>(ss + MR * (MK + 1));
  float* m_s = reinterpret_cast<float*>(ps + MR * prowb);
  float* l_s = m_s + MR;
  float* al_s = l_s + MR;
  int* pos_s = reinterpret_cast<int*>(al_s + MR);
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1], h0 = blockIdx.y * hb;
  const int split = blockIdx.z;
  if (!FMS_IN(seq, a.n_seqs)) return;
  const int slot = a.slots[seq];
  if (!FMS_IN(slot, a.n_slots)) return;
  const int first = first_row[seq] + r0;
  const int ntok = min(tq, first_row[seq + 1] - first);
  if (ntok <= 0) return;
  const int last_pos = ld_fresh(a.positions + first + ntok - 1);
  const int first_pos = ld_fresh(a.positions + first);
  const int seen = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;  // the first key that any row of the tile sees
  const int kt_lo = max(a.n_splits > 1 ? split * (SPLIT / MK) : 0, seen / MK);
  const int n_kt = a.n_splits > 1 ? min(last_pos / MK + 1, (split + 1) * (SPLIT / MK)) : last_pos / MK + 1;
  if (kt_lo >= n_kt) return;  // a split beyond the sequence or before the window: the merge does not look at it
  if (tid < MR) {
    const int tok = tid / hb, hh = tid - tok * hb;
    pos_s[tid] = (tok < ntok && h0 + hh < a.heads) ? ld_fresh(a.positions + first + tok) : -1;
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  const __nv_bfloat16* q = (const __nv_bfloat16*)a.q;
  const __nv_bfloat16* cache = (const __nv_bfloat16*)a.cache;
  const int pieces = width / 8;
  for (int i = tid; i < MR * pieces; i += 256) {
    const int r = i / pieces, piece = i - r * pieces;
    const int tok = r / hb, hh = r - tok * hb;
    const bool ok = tok < ntok && h0 + hh < a.heads;
    lat_copy16(qs + r * rowb + piece * 16, q + ((size_t)(first + (ok ? tok : 0)) * a.heads + (ok ? h0 + hh : 0)) * width + piece * 8, ok);
  }
  auto load_keys = [&](int kt) {
    unsigned char* dst = ks + (kt & 1) * MK * rowb;
    for (int i = tid; i < MK * pieces; i += 256) {
      const int j = i / pieces, piece = i - j * pieces;
      const int p = kt * MK + j;
      int blk = -1;
      if (p <= last_pos) blk = a.table[(size_t)slot * a.table_stride + p / a.block_tokens];
      const bool ok = blk >= 0 && blk < a.n_blocks;
      lat_copy16(dst + j * rowb + piece * 16, cache + ((size_t)(ok ? blk : 0) * a.block_tokens + p % a.block_tokens) * width + piece * 8, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  load_keys(kt_lo);  // one group: the queries and the first keys
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int rg = warp & 1, part = warp >> 1;
  for (int kt = kt_lo; kt < n_kt; ++kt) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // tile kt is in place for everyone, and everyone is done with the other stage
    if (kt + 1 < n_kt) load_keys(kt + 1);
    const unsigned char* kst = ks + (kt & 1) * MK * rowb;
    {  // (A) scores of rows rg * 16 .. + 15 against keys part * 8 .. + 7
      float sacc[4] = {0.f, 0.f, 0.f, 0.f};
      const unsigned char* qrow = qs + (rg * 16 + (lane & 15)) * rowb + (lane >> 4) * 16;
      const unsigned char* krow = kst + (part * 8 + (lane & 7)) * rowb + (lane >> 3) * 16;
      for (int kk = 0; kk < width / 32; ++kk) {
        uint32_t a0[4], a1[4], b[4];
        lat_ldmatrix(a0, qrow + kk * 64);
        lat_ldmatrix(a1, qrow + kk * 64 + 32);
        lat_ldmatrix(b, krow + kk * 64);
        lat_mma(sacc, a0, b[0], b[1]);
        lat_mma(sacc, a1, b[2], b[3]);
      }
      float* dst = ss + (rg * 16 + (lane >> 2)) * (MK + 1) + part * 8 + 2 * (lane & 3);
      dst[0] = sacc[0];
      dst[1] = sacc[1];
      dst[8 * (MK + 1)] = sacc[2];
      dst[8 * (MK + 1) + 1] = sacc[3];
    }
    __syncthreads();
    {  // (B) eight threads a row, four keys each
      const int r = tid >> 3, sub = tid & 7;
      const int pos = pos_s[r];
      const float m_old = m_s[r];
      float sv[4], mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = kt * MK + sub * 4 + j;
        const bool counts = key <= pos && (a.window <= 0 || key > pos - a.window);
        sv[j] = counts ? ss[r * (MK + 1) + sub * 4 + j] * a.scale : -INFINITY;
        mx = fmaxf(mx, sv[j]);
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_old, mx);
      float pv[4], sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pv[j] = m_new == -INFINITY ? 0.f : expf(sv[j] - m_new);
        sum += pv[j];
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __nv_bfloat162* pd = reinterpret_cast<__nv_bfloat162*>(ps + r * prowb + sub * 8);
      pd[0] = __floats2bfloat162_rn(pv[0], pv[1]);
      pd[1] = __floats2bfloat162_rn(pv[2], pv[3]);
      if (sub == 0) {
        const float al = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
        m_s[r] = m_new;
        l_s[r] = l_s[r] * al + sum;
        al_s[r] = al;
      }
    }
    __syncthreads();
    {  // (C) rows rg * 16 .. + 15, columns part * rank / 4 .. of the latent
      const float al0 = al_s[rg * 16 + (lane >> 2)], al1 = al_s[rg * 16 + (lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        acc[i][0] *= al0; acc[i][1] *= al0; acc[i][2] *= al1; acc[i][3] *= al1;
      }
      const int c0 = part * NT * 8;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t pa[4];
        lat_ldmatrix(pa, ps + (rg * 16 + (lane & 15)) * prowb + kk * 32 + (lane >> 4) * 16);
        const unsigned char* vrow = kst + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * rowb + (c0 + (lane >> 4) * 8) * 2;
#pragma unroll
        for (int i = 0; i < NT / 2; ++i) {
          uint32_t b[4];
          lat_ldmatrix_trans(b, vrow + i * 32);
          lat_mma(acc[2 * i], pa, b[0], b[1]);
          lat_mma(acc[2 * i + 1], pa, b[2], b[3]);
        }
      }
    }
  }
  if (a.n_splits > 1) {  // unnormed sums, maximum and sum of this split, for the merge
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = rg * 16 + (lane >> 2) + 8 * half;
      if (pos_s[r] < 0) continue;
      const int tok = r / hb, h = h0 + r - tok * hb;
      const size_t at = ((size_t)(first + tok) * a.heads + h) * a.n_splits + split;
      if (part == 0 && (lane & 3) == 0) {
        a.part_ml[2 * at] = m_s[r];
        a.part_ml[2 * at + 1] = l_s[r];
      }
      float* o = a.part_o + at * a.rank + part * NT * 8 + 2 * (lane & 3);
#pragma unroll
      for (int i = 0; i < NT; ++i) *reinterpret_cast<float2*>(o + i * 8) = make_float2(acc[i][2 * half], acc[i][2 * half + 1]);
    }
    return;
  }
  __syncthreads();
  if (tid < MR) {  // what each row's sums are multiplied by: the softmax's denominator with the sink, and the gate
    float f = 0.f;
    if (pos_s[tid] >= 0) {
      const int tok = tid / hb, h = h0 + tid - tok * hb;
      float m = m_s[tid], denom = l_s[tid], top = m;
      if (a.sink) {
        const float sk = to_f32(((const TS*)a.sink)[h]);
        top = fmaxf(m, sk);
        denom = denom * expf(m - top) + expf(sk - top);
      }
      f = expf(m - top) / denom;
      if (a.gate) f *= 1.f / (1.f + expf(-to_f32(((const __nv_bfloat16*)a.gate)[(size_t)(first + tok) * a.gate_stride + h])));
    }
    al_s[tid] = f;
  }
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = rg * 16 + (lane >> 2) + 8 * half;
    if (pos_s[r] < 0) continue;
    const int tok = r / hb, h = h0 + r - tok * hb;
    const float f = al_s[r];
    __nv_bfloat16* o = (__nv_bfloat16*)a.out + ((size_t)(first + tok) * a.heads + h) * a.rank + part * NT * 8 + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < NT; ++i)
      *reinterpret_cast<__nv_bfloat162*>(o + i * 8) = __floats2bfloat162_rn(acc[i][2 * half] * f, acc[i][2 * half + 1] * f);
  }
}

template <typename T, typename TS>
int launch_attention(const LatentArgs& a, int n_tokens, cudaStream_t stream) {
  const int width = a.rank + a.rot;
  const size_t smem = ((size_t)HG * width + (size_t)KT * (width | 1) + HG * KT + HG) * sizeof(float);
  if (smem > 220 * 1024) return fms_fail("latent_attention: rows of %d values do not fit shared memory", width);
  if (a.block_tokens % KT) return fms_fail("latent_attention: cache blocks of %d tokens", a.block_tokens);
  dim3 grid(n_tokens, a.n_splits, (a.heads + HG - 1) / HG);
  if (grid.y > 65535 || grid.z > 65535) return fms_fail("latent_attention: %d splits, %d heads", a.n_splits, a.heads);
#define FMS_LATENT_LAUNCH(NACC)                                                                                         \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(latent_attention_kernel<T, TS, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    fms_launch(latent_attention_kernel<T, TS, NACC>, grid, dim3(THREADS), smem, stream, a);                             \
  } while (0)
  if (a.rank <= 128) FMS_LATENT_LAUNCH(4);
  else if (a.rank <= 256) FMS_LATENT_LAUNCH(8);
  else if (a.rank <= 512) FMS_LATENT_LAUNCH(16);
  else if (a.rank <= 1024) FMS_LATENT_LAUNCH(32);
  else return fms_fail("latent_attention: a latent of %d values is more than the kernel keeps (1024)", a.rank);
#undef FMS_LATENT_LAUNCH
  if (fms_launch_status("latent_attention")) return 1;
  if (a.n_splits > 1) {
    fms_launch(latent_combine_kernel<T, TS>, dim3(n_tokens, a.heads), dim3(128), 0, stream, a);
    return fms_launch_status("latent_attention (combine)");
  }
  return 0;
}
}  // namespace

FMS_API int fms_latent_split_tokens() { return SPLIT; }

// x: the first of the n columns to norm in row 0 of a matrix with rows of `stride` values; out [n_tokens, n]
FMS_API int fms_latent_query_norm(const void* x, int dtype, int stride, int n, const void* gain, int gain_dtype, float eps,
                                  void* out, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n <= 0 || stride < n) return fms_fail("latent_query_norm: %d columns of rows of %d", n, stride);
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  const int vec = n % 4 == 0 && stride % 4 == 0 && (uintptr_t)x % (4 * item) == 0;
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(latent_query_norm_kernel<T, TG>, dim3(n_tokens), dim3(128), 0, stream, (const T*)x,
                                stride, n, (const TG*)gain, eps, (T*)out, n_tokens, vec)));
  return fms_launch_status("latent_query_norm");
}

FMS_API int fms_latent_prepare(const void* proj, int dtype, int proj_width, void* q_full, const void* c_gain, int gain_dtype,
                               float eps, const float* inv_freq, int rot_dims, const int* positions,
                               const int* position_ids, const int* token_seq, const int* slots, void* cache,
                               const int* table, int table_stride, int block_tokens, int n_tokens, int heads, int dim,
                               int rot, int rank, int write_cache, int n_seqs, int n_slots, int n_blocks, int* error_flag,
                               int halves, float rot_mult, const void* kv, int kv_width, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || dim < 0 || rot < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1))
    return fms_fail("latent_prepare: heads %d, dim %d, rot %d (%d rotated), rank %d", heads, dim, rot, rot_dims, rank);
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(latent_prepare_kernel<T, TG>, dim3(n_tokens), dim3(128), 0, stream, (const T*)proj,
                                proj_width, (T*)q_full, (const TG*)c_gain, eps, inv_freq, rot_dims, positions,
                                position_ids, token_seq, slots, (T*)cache, table, table_stride, block_tokens, heads, dim,
                                rot, rank, write_cache, n_seqs, n_slots, n_blocks, error_flag, halves, rot_mult,
                                (const T*)kv, kv_width)));
  return fms_launch_status("latent_prepare");
}

// n_splits == 1: every row takes all its keys in one block (a prompt's rows); else splits of fms_latent_split_tokens()
// keys and a merge, with part_o [tokens, heads, splits, rank] and part_ml [tokens, heads, splits, 2] as scratch.
FMS_API int fms_latent_attention(const void* q, void* out, int dtype, const void* cache, const void* gate, long gate_stride,
                                 const void* sink, int sink_dtype, const int* table, int table_stride, int block_tokens,
                                 const int* slots, const int* token_seq, const int* positions, int n_tokens, int n_splits,
                                 float* part_o, float* part_ml, int heads, int rank, int rot, float scale, int n_seqs,
                                 int n_slots, int n_blocks, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_splits < 1 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
    return fms_fail("latent_attention: %d splits without scratch", n_splits);
  LatentArgs a;
  a.q = q; a.out = out; a.cache = cache; a.gate = gate; a.sink = sink; a.table = table; a.slots = slots;
  a.token_seq = token_seq; a.positions = positions; a.part_o = part_o; a.part_ml = part_ml; a.gate_stride = gate_stride;
  a.table_stride = table_stride; a.block_tokens = block_tokens; a.heads = heads; a.rank = rank; a.rot = rot;
  a.n_splits = n_splits; a.n_seqs = n_seqs; a.n_slots = n_slots; a.n_blocks = n_blocks; a.scale = scale;
  a.window = window > 0 ? window : 0;
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(sink ? sink_dtype : dtype, TS, return launch_attention<T, TS>(a, n_tokens, stream)));
  return 0;
}

// Many rows of bfloat16 on the tensor cores: rank a multiple of 64 up to 512, rank + rot a multiple of 32.  tiles
// [n_tiles, 2] = (sequence, first of its `tile_tokens` rows within the sequence's rows of this step); a block takes
// tile_tokens tokens times heads_per_block heads, tile_tokens * heads_per_block = 32.
FMS_API int fms_latent_attention_prefill_bf16(const void* q, void* out, const void* cache, const void* gate, long gate_stride,
                                              const void* sink, int sink_dtype, const int* table, int table_stride,
                                              int block_tokens, const int* slots, const int* first_row,
                                              const int* positions, const int* tiles, int n_tiles, int tile_tokens,
                                              int heads_per_block, int heads, int rank, int rot, float scale, int n_seqs,
                                              int n_slots, int n_blocks, const int* token_seq, int n_splits, float* part_o,
                                              float* part_ml, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (n_splits < 1 || (n_splits > 1 && (tile_tokens != 1 || part_o == nullptr || part_ml == nullptr || token_seq == nullptr)))
    return fms_fail("latent_attention_prefill: %d splits need one token a tile and scratch", n_splits);
  const int width = rank + rot;
  if (rank % 64 || rank > 512 || width % 32 || tile_tokens * heads_per_block != MR)
    return fms_fail("latent_attention_prefill: rank %d, rot %d, %d tokens x %d heads a block", rank, rot, tile_tokens, heads_per_block);
  LatentArgs a;
  a.q = q; a.out = out; a.cache = cache; a.gate = gate; a.sink = sink; a.table = table; a.slots = slots;
  a.token_seq = token_seq; a.positions = positions; a.part_o = part_o; a.part_ml = part_ml; a.gate_stride = gate_stride;
  a.table_stride = table_stride; a.block_tokens = block_tokens; a.heads = heads; a.rank = rank; a.rot = rot;
  a.n_splits = n_splits; a.n_seqs = n_seqs; a.n_slots = n_slots; a.n_blocks = n_blocks; a.scale = scale;
  a.window = window > 0 ? window : 0;
  const int rowb = width * 2 + 16;
  const size_t smem = (size_t)(MR + 2 * MK) * rowb + MR * (MK + 1) * 4 + MR * (MK * 2 + 16) + MR * 16;
  dim3 grid(n_tiles, (heads + heads_per_block - 1) / heads_per_block, n_splits);
  if (grid.z > 65535) return fms_fail("latent_attention_prefill: %d splits", n_splits);
#define FMS_LATENT_MMA(NT)                                                                                              \
  case NT:                                                                                                              \
    if (sink && sink_dtype == FMS_F32) {                                                                                \
      cudaFuncSetAttribute(latent_prefill_mma_kernel<float, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      fms_launch(latent_prefill_mma_kernel<float, NT>, grid, dim3(256), smem, stream, a, tiles, first_row, tile_tokens,   \
                 heads_per_block);                                                                                      \
    } else {                                                                                                            \
      cudaFuncSetAttribute(latent_prefill_mma_kernel<__nv_bfloat16, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                           (int)smem);                                                                                  \
      fms_launch(latent_prefill_mma_kernel<__nv_bfloat16, NT>, grid, dim3(256), smem, stream, a, tiles, first_row,       \
                 tile_tokens, heads_per_block);                                                                         \
    }                                                                                                                   \
    break;
  switch (rank / 32) {
    FMS_LATENT_MMA(2) FMS_LATENT_MMA(4) FMS_LATENT_MMA(6) FMS_LATENT_MMA(8) FMS_LATENT_MMA(10) FMS_LATENT_MMA(12)
    FMS_LATENT_MMA(14) FMS_LATENT_MMA(16)
    default: return fms_fail("latent_attention_prefill: rank %d", rank);
  }
#undef FMS_LATENT_MMA
  if (fms_launch_status("latent_attention_prefill")) return 1;
  if (n_splits > 1) {  // one token a tile: the rows of the merge are the step's rows, tile i being row i
    if (sink && sink_dtype == FMS_F32)
      fms_launch(latent_combine_kernel<__nv_bfloat16, float>, dim3(n_tiles, heads), dim3(128), 0, stream, a);
    else
      fms_launch(latent_combine_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(n_tiles, heads), dim3(128), 0, stream, a);
    return fms_launch_status("latent_attention (combine)");
  }
  return 0;
}
