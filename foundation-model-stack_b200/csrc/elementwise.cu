// Memory-bound kernels of a decoder step: embedding rows, residual add + RMSNorm in one pass, gated
// activation, and rotary position encoding fused with the write of keys and values into the block cache.
// All arithmetic is float32; inputs and outputs are float32 or bfloat16.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------
// embedding: out[t, :] = scale * float(table[tokens[t], :])    (reference: fms/models/llama.py:332; scale 1)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void embed_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void embed_load8(const __nv_bfloat16* p, float* v) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __uint_as_float(w[k] << 16);
    v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out,
                                  int dim, int vocab, float scale, int* __restrict__ error_flag) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  const T* src = table + (size_t)(ok ? tok : 0) * dim;
  float* dst = out + (size_t)t * dim;
  if ((dim & 7) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    // 8 values a thread and step: 16 bytes in for bfloat16 (two loads for float32), two 16-byte stores out
    for (int d = 8 * threadIdx.x; d < dim; d += 8 * blockDim.x) {
      float v[8];
      embed_load8(src + d, v);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (ok) {
        a = make_float4(scale * v[0], scale * v[1], scale * v[2], scale * v[3]);
        b = make_float4(scale * v[4], scale * v[5], scale * v[6], scale * v[7]);
      }
      *reinterpret_cast<float4*>(dst + d) = a;
      *reinterpret_cast<float4*>(dst + d + 4) = b;
    }
    return;
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = ok ? scale * to_f32(src[d]) : 0.f;
}

FMS_API int fms_embed_rows(const void* table, int table_dtype, const int* tokens, float* out, int n_tokens, int dim,
                           int vocab, float scale, int* error_flag, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || vocab <= 0) return fms_fail("embed_rows: dim %d, vocab %d", dim, vocab);
  const int threads = dim >= 1024 ? 256 : 128;
  FMS_DISPATCH_DTYPE(table_dtype, T,
                     fms_launch(embed_rows_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)table, tokens,
                                out, dim, vocab, scale, error_flag));
  return fms_launch_status("embed_rows");
}

// ---------------------------------------------------------------------------------------------------
// embedding with a hashed table of token pairs beside the token table:
//   out[t, :] = scale * (float(table[tokens[t]]) + float(pairs[row(t)]))
//   row(t) = (previous * mul_prev + tokens[t] * mul_cur) mod buckets, or `buckets` (the table's last row) for the token
//   at place 0 of its sequence.  The previous token of a step's first row comes from the sequence's state
//   (last_token[slot], one int per slot), which the block of that row then sets to the step's last token of the
//   sequence: no other block touches it.  64-bit integer arithmetic.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_pair_hash_kernel(const T* table, const T* pairs,
                                       const int* tokens, const int* positions,
                                       const int* token_seq, const int* first_row,
                                       const int* slots, int* last_token,
                                       float* out, int dim, int vocab, long long buckets,
                                       long long mul_prev, long long mul_cur, float scale, int update_state,
                                       int n_seqs, int n_slots, int* error_flag) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int slot = slots[seq], first = first_row[seq];
  if (!FMS_IN(slot, n_slots)) return;
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  long long row = buckets;
  if (__ldcg(positions + t) != 0) {  // written by the kernel right before this one in a decode step
    const long long prev = t == first ? last_token[slot] : tokens[t - 1];
    row = (prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  if (t == first && update_state) {
    __syncthreads();  // every thread of this block has read the state
    if (threadIdx.x == 0) last_token[slot] = tokens[first_row[seq + 1] - 1];
  }
  const T* src = table + (size_t)(ok ? tok : 0) * dim;
  const T* two = pairs + (size_t)(ok ? row : buckets) * dim;
  float* dst = out + (size_t)t * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = ok ? scale * (to_f32(src[d]) + to_f32(two[d])) : 0.f;
}

FMS_API int fms_embed_pair_hash(const void* table, const void* pairs, int table_dtype, const int* tokens,
                                const int* positions, const int* token_seq, const int* first_row, const int* slots,
                                int* last_token, float* out, int n_tokens, int dim, int vocab, long buckets, long mul_prev,
                                long mul_cur, float scale, int update_state, int n_seqs, int n_slots, int* error_flag,
                                cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || vocab <= 0 || buckets <= 0) return fms_fail("embed_pair_hash: dim %d, vocab %d, buckets %ld", dim, vocab, buckets);
  const int threads = dim >= 1024 ? 256 : 128;
  FMS_DISPATCH_DTYPE(table_dtype, T,
                     fms_launch(embed_pair_hash_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)table,
                                (const T*)pairs, tokens, positions, token_seq, first_row, slots, last_token, out, dim,
                                vocab, (long long)buckets, (long long)mul_prev, (long long)mul_cur, scale, update_state,
                                n_seqs, n_slots, error_flag));
  return fms_launch_status("embed_pair_hash");
}

// ---------------------------------------------------------------------------------------------------
// residual add + RMSNorm                                     (reference: fms/modules/layernorm.py:56-69)
//   x = residual[src] + delta[src]       float32; written back to residual unless rows are gathered
//   out[r] = gain * x * rsqrt(mean(x^2) + eps)
// One thread block per output row; the row is read twice (the second time from cache).
// ---------------------------------------------------------------------------------------------------
template <typename T, typename TG>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const TG* __restrict__ gain, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
  float ss = 0.f;
  if (rows == nullptr) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      float x = res[d];
      if (del) {
        x += to_f32(del[d]);
        res[d] = x;
      }
      ss += x * x;
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      float x = res[d] + (del ? to_f32(del[d]) : 0.f);
      ss += x * x;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)dim + eps);
  T* o = out + (size_t)r * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float x = res[d];
    if (rows != nullptr && del) x += to_f32(del[d]);
    o[d] = from_f32<T>(to_f32(gain[d]) * (x * inv));
  }
}

// The same for rows whose width is a multiple of 4 and at most 4 * NCHUNK * blockDim: each thread keeps its
// part of the row in registers, all loads are issued before the first store, nothing is read twice.
__device__ __forceinline__ void load4(const float* p, float* v) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename T, typename TG, int NCHUNK>
__global__ void add_rmsnorm_regs_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const TG* __restrict__ gain, float eps, T* __restrict__ out,
                                        const int* __restrict__ rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int nvec = dim >> 2;
  float x[NCHUNK][4], dl[NCHUNK][4], g[NCHUNK][4];
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {  // the gain is a weight: it can be read before the kernel before this one is done
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) load4(gain + 4 * c, g[j]);
  }
  pdl_wait();
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      load4(res + 4 * c, x[j]);
      if (del) load4(del + 4 * c, dl[j]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (del) x[j][e] += dl[j][e];
        ss += x[j][e] * x[j][e];
      }
      if (del && rows == nullptr) store4(res + 4 * c, x[j]);
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)dim + eps);
  T* o = out + (size_t)r * dim;
#pragma unroll
  for (int j = 0; j < NCHUNK; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = g[j][e] * (x[j][e] * inv);
      store4(o + 4 * c, y);
    }
  }
}

// residual_rows: rows of the residual stream (and of delta), which the entries of `rows` index; used by the
// bounds-checked build only (0: not known)
FMS_API int fms_add_rmsnorm(float* residual, const void* delta, const void* gain, int gain_dtype, float eps, void* out,
                            int dtype, const int* rows, int n_rows, int dim, int residual_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return fms_fail("add_rmsnorm: dim %d", dim);
  if (dim % 4 == 0 && dim <= 4 * 4 * 1024) {
    // up to 4 chunks of 4 values per thread; few rows: more threads per row, so that each has one chunk
    const int nvec = dim / 4;
    int threads = 128;
    while (threads < 1024 && threads * (n_rows <= 64 ? 1 : 4) < nvec) threads *= 2;
    const int nchunk = (nvec + threads - 1) / threads;
    FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG, {
      if (nchunk <= 1)
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 1>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
      else if (nchunk <= 2)
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 2>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
      else
        fms_launch(add_rmsnorm_regs_kernel<T, TG, 4>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   (const TG*)gain, eps, (T*)out, rows, dim, residual_rows);
    }));
    return fms_launch_status("add_rmsnorm");
  }
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(add_rmsnorm_kernel<T, TG>, dim3(n_rows), dim3(threads), 0, stream, residual,
                                (const T*)delta, (const TG*)gain, eps, (T*)out, rows, dim, residual_rows)));
  return fms_launch_status("add_rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// a sublayer's output normed on its way into the residual stream, and the next norm, in one pass over the row:
//   d = delta * (1 / sqrt(mean(delta^2) + post_eps)) * post_gain        (skipped where has_post == 0: d = delta)
//   x = residual[src] + d                 float32; written back to residual unless rows are gathered
//   out[r] = x * (1 / sqrt(mean(x^2) + eps)) * gain
// Each gain is one number for the whole row (the vector pointer null) or a vector of `dim`.  One block per row.
// ---------------------------------------------------------------------------------------------------
template <typename T, typename TG>
__global__ void normed_add_rmsnorm_kernel(float* residual, const T* delta, int has_post,
                                          const TG* post_gain_vec, float post_gain, float post_eps,
                                          const TG* gain_vec, float gain, float eps, T* out,
                                          const int* rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
  float inv_d = 1.f;
  if (del && has_post) {
    float sd = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float v = to_f32(del[d]);
      sd += v * v;
    }
    inv_d = 1.f / sqrtf(block_sum(sd, scratch) / (float)dim + post_eps);
  }
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float x = res[d];
    if (del) {
      float v = to_f32(del[d]);
      if (has_post) v = v * inv_d * (post_gain_vec ? to_f32(post_gain_vec[d]) : post_gain);
      x += v;
      if (rows == nullptr) res[d] = x;
    }
    ss += x * x;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  T* o = out + (size_t)r * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float x = res[d];  // this thread's own earlier store, where the sum was written back
    if (rows != nullptr && del) {
      float v = to_f32(del[d]);
      if (has_post) v = v * inv_d * (post_gain_vec ? to_f32(post_gain_vec[d]) : post_gain);
      x += v;
    }
    o[d] = from_f32<T>(x * inv * (gain_vec ? to_f32(gain_vec[d]) : gain));
  }
}

// The same with the row in registers: NPER values a thread (dim <= NPER * blockDim), every value read once.
template <typename T, typename TG, int NPER>
__global__ void normed_add_rmsnorm_regs_kernel(float* residual, const T* delta, int has_post, const TG* post_gain_vec,
                                               float post_gain, float post_eps, const TG* gain_vec, float gain, float eps,
                                               T* out, const int* rows, int dim, int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  const T* del = delta ? delta + (size_t)src * dim : nullptr;
  float x[NPER], v[NPER];
  float sd = 0.f;
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    x[j] = d < dim ? res[d] : 0.f;
    v[j] = (del && d < dim) ? to_f32(del[d]) : 0.f;
    sd += v[j] * v[j];
  }
  float inv_d = 1.f;
  if (del && has_post) inv_d = 1.f / sqrtf(block_sum(sd, scratch) / (float)dim + post_eps);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    if (d < dim && del) {
      float add = v[j];
      if (has_post) add = add * inv_d * (post_gain_vec ? to_f32(post_gain_vec[d]) : post_gain);
      x[j] += add;
      if (rows == nullptr) res[d] = x[j];
    }
    ss += x[j] * x[j];
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  T* o = out + (size_t)r * dim;
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    if (d < dim) o[d] = from_f32<T>(x[j] * inv * (gain_vec ? to_f32(gain_vec[d]) : gain));
  }
}

FMS_API int fms_normed_add_rmsnorm(float* residual, const void* delta, int has_post, const void* post_gain_vec,
                                   float post_gain, float post_eps, const void* gain_vec, float gain, float eps,
                                   int gain_dtype, void* out, int dtype, const int* rows, int n_rows, int dim,
                                   int residual_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return fms_fail("normed_add_rmsnorm: dim %d", dim);
  const int threads = dim >= 4096 ? 1024 : (dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128));
  if (dim <= 8 * threads) {  // the row fits the block's registers
    const int nper = (dim + threads - 1) / threads;
    FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG, {
      if (nper <= 2)
        fms_launch(normed_add_rmsnorm_regs_kernel<T, TG, 2>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   has_post, (const TG*)post_gain_vec, post_gain, post_eps, (const TG*)gain_vec, gain, eps, (T*)out, rows, dim,
                   residual_rows);
      else if (nper <= 4)
        fms_launch(normed_add_rmsnorm_regs_kernel<T, TG, 4>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   has_post, (const TG*)post_gain_vec, post_gain, post_eps, (const TG*)gain_vec, gain, eps, (T*)out, rows, dim,
                   residual_rows);
      else
        fms_launch(normed_add_rmsnorm_regs_kernel<T, TG, 8>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta,
                   has_post, (const TG*)post_gain_vec, post_gain, post_eps, (const TG*)gain_vec, gain, eps, (T*)out, rows, dim,
                   residual_rows);
    }));
    return fms_launch_status("normed_add_rmsnorm");
  }
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(normed_add_rmsnorm_kernel<T, TG>, dim3(n_rows), dim3(threads), 0, stream, residual,
                                (const T*)delta, has_post, (const TG*)post_gain_vec, post_gain, post_eps,
                                (const TG*)gain_vec, gain, eps, (T*)out, rows, dim, residual_rows)));
  return fms_launch_status("normed_add_rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// The same step for norms of either kind, each chosen by a mode: 0 none, 1 root mean square, 2 layer norm (the mean is
// taken off first and the variance is the mean of the squared deviations; no bias).  Gains are float32 vectors of
// `dim` (a layer scale that multiplies a norm's result is folded into its gain by the caller):
//   d = post(delta) * post_gain                              post_mode 0: d = delta
//   x = residual[src] + d                float32; written back to residual unless rows are gathered
//   out[r] = norm(x) * gain                                   out_mode 0: out[r] = x, the stream in the compute dtype
//                                                             (no out pointer: nothing but the sum is wanted)
// A block per row with the row in registers, NPER values a thread (dim <= NPER * blockDim).
// ---------------------------------------------------------------------------------------------------
template <int NPER>
__device__ __forceinline__ void norm_in_registers(float (&v)[NPER], int mode, const float* gain_vec, float eps, int dim,
                                                  float* scratch) {
  if (mode == 0) return;
  float mean = 0.f;
  if (mode == 2) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NPER; ++j) sum += v[j];  // values beyond the row are zeros
    mean = block_sum(sum, scratch) / (float)dim;
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    const float c = d < dim ? v[j] - mean : 0.f;
    v[j] = c;
    ss += c * c;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    if (d < dim) v[j] = v[j] * inv * gain_vec[d];
  }
}

template <typename T, int NPER>
__global__ void normed_add_norm_kernel(float* residual, const T* delta, int post_mode, const float* post_gain, float post_eps,
                                       int out_mode, const float* gain, float eps, T* out, const int* rows, int dim,
                                       int residual_rows) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (!FMS_IN(src, residual_rows)) return;  // the whole block alike
  float* res = residual + (size_t)src * dim;
  float x[NPER];
  if (delta) {
    const T* del = delta + (size_t)src * dim;
    float v[NPER];
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int d = threadIdx.x + j * blockDim.x;
      v[j] = d < dim ? to_f32(del[d]) : 0.f;
    }
    norm_in_registers<NPER>(v, post_mode, post_gain, post_eps, dim, scratch);
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int d = threadIdx.x + j * blockDim.x;
      x[j] = d < dim ? res[d] + v[j] : 0.f;
      if (d < dim && rows == nullptr) res[d] = x[j];
    }
  } else {
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int d = threadIdx.x + j * blockDim.x;
      x[j] = d < dim ? res[d] : 0.f;
    }
  }
  if (out == nullptr) return;
  norm_in_registers<NPER>(x, out_mode, gain, eps, dim, scratch);
  T* o = out + (size_t)r * dim;
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int d = threadIdx.x + j * blockDim.x;
    if (d < dim) o[d] = from_f32<T>(x[j]);
  }
}

FMS_API int fms_normed_add_norm(float* residual, const void* delta, int post_mode, const float* post_gain, float post_eps,
                                int out_mode, const float* gain, float eps, void* out, int dtype, const int* rows,
                                int n_rows, int dim, int residual_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0 || dim > 16384) return fms_fail("normed_add_norm: rows of %d values (up to 16384)", dim);
  if (post_mode < 0 || post_mode > 2 || out_mode < 0 || out_mode > 2) return fms_fail("normed_add_norm: modes %d, %d", post_mode, out_mode);
  if ((post_mode && delta && !post_gain) || (out_mode && out && !gain)) return fms_fail("normed_add_norm: a norm without its gain");
  const int threads = dim >= 4096 ? 1024 : (dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128));
  const int nper = (dim + threads - 1) / threads;
#define FMS_NAN(NPER)                                                                                                     \
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(normed_add_norm_kernel<T, NPER>, dim3(n_rows), dim3(threads), 0, stream, residual,   \
                                          (const T*)delta, post_mode, post_gain, post_eps, out_mode, gain, eps, (T*)out, rows, \
                                          dim, residual_rows))
  if (nper <= 2) FMS_NAN(2);
  else if (nper <= 4) FMS_NAN(4);
  else if (nper <= 8) FMS_NAN(8);
  else FMS_NAN(16);
#undef FMS_NAN
  return fms_launch_status("normed_add_norm");
}

// ---------------------------------------------------------------------------------------------------
// gated activation: out[n, f] = act(gu[n, f]) * gu[n, hidden + f]   (fms/modules/feedforward.py:291-292)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float activate(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + expf(-g));                                               // silu
    case 1: return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));                  // gelu
    case 2: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));  // gelu-tanh
    default: return fmaxf(g, 0.f);                                                     // relu
  }
}

template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gu, T* __restrict__ out, int hidden, int act,
                                        size_t total) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t n = i / hidden;
    const int f = (int)(i - n * hidden);
    const float g = to_f32(gu[n * 2 * hidden + f]);
    const float u = to_f32(gu[n * 2 * hidden + hidden + f]);
    out[i] = from_f32<T>(activate(g, act) * u);
  }
}

// bfloat16 rows whose width is a multiple of 8: 8 values (16 bytes) of gate and of up per thread
__global__ void gated_activation_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                            int hidden, int act, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = hidden >> 3;
  const long total = (long)n_rows * per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int n = (int)(i / per_row), f = (int)(i - (long)n * per_row) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)n * 2 * hidden + f);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)n * 2 * hidden + hidden + f);
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
      const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
      __nv_bfloat162 r = __floats2bfloat162_rn(activate(g0, act) * u0, activate(g1, act) * u1);
      ow[k] = *reinterpret_cast<uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * hidden + f) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

FMS_API int fms_gated_activation(const void* gu, void* out, int dtype, int n_rows, int hidden, int act,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || act < 0 || act > 3) return fms_fail("gated_activation: hidden %d, act %d", hidden, act);
  const int threads = 256;
  if (dtype == FMS_BF16 && hidden % 8 == 0) {
    const long total = (long)n_rows * (hidden / 8);
    const int blocks = (int)((total + threads - 1) / threads < 148 * 32 ? (total + threads - 1) / threads : 148 * 32);
    fms_launch(gated_activation_vec_kernel, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gu,
               (__nv_bfloat16*)out, hidden, act, n_rows);
    return fms_launch_status("gated_activation");
  }
  const size_t total = (size_t)n_rows * hidden;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  FMS_DISPATCH_DTYPE(dtype, T,
                     gated_activation_kernel<T><<<blocks, threads, 0, stream>>>((const T*)gu, (T*)out, hidden, act,
                                                                                total));
  return fms_launch_status("gated_activation");
}

// ---------------------------------------------------------------------------------------------------
// rotary encoding + cache write
//   qkv[t] = [q heads | k heads | v heads], each head `head_dim` wide     (fms/modules/attention.py:653-657)
//   q, k: adjacent pairs (2i, 2i+1) rotated by angle = position * inv_freq[i], float32
//                                                                    (fms/modules/positions.py:438-456)
//   positions[t]: the token's place in its sequence's cache; position_ids[t]: the position that the rotation sees
//   (null: the same; they differ for a sequence that does not start at position 0)
//   rotated q -> q_out[t]; rotated k and v -> the cache block of the token's slot and position
// grid (token, head), one thread per pair.
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ inv_freq,
                                  const int* __restrict__ positions, const int* __restrict__ position_ids,
                                  const int* __restrict__ token_seq,
                                  const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ table, int table_stride, int block_tokens, int nheads,
                                  int kvheads, int head_dim, int write_cache, int* __restrict__ error_flag, int n_seqs,
                                  int table_rows, int pool_blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..nheads-1: q; then k heads; then v heads
  const int i = threadIdx.x;    // pair index
  if (i >= head_dim / 2) return;
  const int pos = positions[t];
  const int width = (nheads + 2 * kvheads) * head_dim;
  const T* src = qkv + (size_t)t * width + (size_t)head * head_dim;
  float x0 = to_f32(src[2 * i]), x1 = to_f32(src[2 * i + 1]);
  const bool is_v = head >= nheads + kvheads;
  if (!is_v && inv_freq != nullptr) {
    const float angle = (float)(position_ids ? position_ids[t] : pos) * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    const float r0 = c * x0 - s * x1;
    const float r1 = s * x0 + c * x1;
    x0 = r0;
    x1 = r1;
  }
  if (head < nheads) {
    T* dst = q_out + (size_t)t * nheads * head_dim + (size_t)head * head_dim;
    dst[2 * i] = from_f32<T>(x0);
    dst[2 * i + 1] = from_f32<T>(x1);
    return;
  }
  if (!write_cache) return;
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, table_rows) || !FMS_IN(pos / block_tokens, table_stride)) return;
  const int blk = table[(size_t)slot * table_stride + pos / block_tokens];
  if (blk < 0) {
    if (i == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  if (!FMS_IN(blk, pool_blocks)) return;
  const int kvh = is_v ? head - nheads - kvheads : head - nheads;
  T* base = is_v ? v_cache : k_cache;
  T* dst = base + (((size_t)blk * kvheads + kvh) * block_tokens + (pos % block_tokens)) * head_dim;
  dst[2 * i] = from_f32<T>(x0);
  dst[2 * i + 1] = from_f32<T>(x1);
}

// bfloat16, many tokens: one block per token, a thread per 16-byte piece (8 values = 4 pairs) of a head.  The
// angle of a pair is the same for every head of the token: its sine and cosine are taken once, into shared memory.
constexpr int ROPE_VEC_MAX_PAIRS = 1024;  // head_dim / 2 that the table in shared memory holds

__global__ void rope_store_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ position_ids, const int* __restrict__ token_seq,
                                      const int* __restrict__ slots,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      const int* __restrict__ table, int table_stride, int block_tokens, int nheads,
                                      int kvheads, int head_dim, int write_cache, int* __restrict__ error_flag,
                                      int n_seqs, int table_rows, int pool_blocks) {
  extern __shared__ float2 sincos_of_pair[];  // [head_dim / 2]: (sin, cos)
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int pieces = head_dim >> 3;
  const int total = (nheads + 2 * kvheads) * pieces;
  const size_t width = (size_t)(nheads + 2 * kvheads) * head_dim;
  int blk = 0;
  if (write_cache) {
    const int seq = token_seq[t];
    const int slot = FMS_IN(seq, n_seqs) ? slots[seq] : -1;
    if (slot >= 0 && FMS_IN(slot, table_rows) && FMS_IN(pos / block_tokens, table_stride)) {
      blk = table[(size_t)slot * table_stride + pos / block_tokens];
      if (blk < 0 && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
      if (blk >= 0 && !FMS_IN(blk, pool_blocks)) blk = -1;
    } else {
      blk = -1;
    }
  }
  if (inv_freq != nullptr) {
    const float turned_by = (float)(position_ids ? position_ids[t] : pos);
    for (int i = threadIdx.x; i < head_dim / 2; i += blockDim.x) {
      float sn, cs;
      sincosf(turned_by * inv_freq[i], &sn, &cs);
      sincos_of_pair[i] = make_float2(sn, cs);
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int head = i / pieces, piece = i - head * pieces;
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + (size_t)t * width + (size_t)head * head_dim + piece * 8);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const bool is_v = head >= nheads + kvheads;
    if (!is_v && inv_freq != nullptr) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x0 = __uint_as_float(w[k] << 16), x1 = __uint_as_float(w[k] & 0xffff0000u);
        const float2 sc = sincos_of_pair[piece * 4 + k];
        __nv_bfloat162 r = __floats2bfloat162_rn(sc.y * x0 - sc.x * x1, sc.x * x0 + sc.y * x1);
        w[k] = *reinterpret_cast<uint32_t*>(&r);
      }
    }
    const uint4 o = make_uint4(w[0], w[1], w[2], w[3]);
    if (head < nheads) {
      *reinterpret_cast<uint4*>(q_out + ((size_t)t * nheads + head) * head_dim + piece * 8) = o;
    } else if (write_cache && blk >= 0) {
      const int kvh = is_v ? head - nheads - kvheads : head - nheads;
      __nv_bfloat16* base = is_v ? v_cache : k_cache;
      *reinterpret_cast<uint4*>(base + (((size_t)blk * kvheads + kvh) * block_tokens + (pos % block_tokens)) * head_dim +
                                piece * 8) = o;
    }
  }
}

FMS_API int fms_rope_store(const void* qkv, int dtype, void* q_out, const float* inv_freq, const int* positions,
                           const int* position_ids, const int* token_seq, const int* slots, void* k_cache, void* v_cache, const int* table,
                           int table_stride, int block_tokens, int n_tokens, int nheads, int kvheads, int head_dim,
                           int write_cache, int* error_flag, int n_seqs, int table_rows, int pool_blocks,
                           cudaStream_t stream) {
  // n_seqs, table_rows, pool_blocks: extents of slots, of the table and of the cache, for the bounds-checked build (0: not known)
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim % 2 || head_dim > 2048) return fms_fail("rope_store: head_dim %d", head_dim);
  if (dtype == FMS_BF16 && head_dim % 8 == 0 && n_tokens >= 64 && head_dim / 2 <= ROPE_VEC_MAX_PAIRS) {
    const int total = (nheads + 2 * kvheads) * (head_dim / 8);
    const int threads = total >= 256 ? 256 : ((total + 31) / 32) * 32;
    fms_launch(rope_store_vec_kernel, dim3(n_tokens), dim3(threads), (size_t)(head_dim / 2) * sizeof(float2), stream,
               (const __nv_bfloat16*)qkv,
               (__nv_bfloat16*)q_out, inv_freq, positions, position_ids, token_seq, slots, (__nv_bfloat16*)k_cache,
               (__nv_bfloat16*)v_cache, table, table_stride, block_tokens, nheads, kvheads, head_dim, write_cache,
               error_flag, n_seqs, table_rows, pool_blocks);
    return fms_launch_status("rope_store");
  }
  dim3 grid(n_tokens, nheads + 2 * kvheads);
  const int threads = ((head_dim / 2 + 31) / 32) * 32;
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(rope_store_kernel<T>, grid, dim3(threads), 0, stream, (const T*)qkv, (T*)q_out, inv_freq,
                                positions, position_ids, token_seq, slots, (T*)k_cache, (T*)v_cache, table, table_stride,
                                block_tokens,
                                nheads, kvheads, head_dim, write_cache, error_flag, n_seqs, table_rows, pool_blocks));
  return fms_launch_status("rope_store");
}

// ---------------------------------------------------------------------------------------------------
// (sin, cos) of every token's rotation angles, once a step for all layers that rotate by the same frequencies:
//   out[t, i] = (sin, cos)(position(t) * inv_freq[i]),  position = position_ids[t] if given, else positions[t]
// the float32 product and sincosf of the rotation kernels themselves, so a kernel that reads the table turns by the
// very angles one that takes them itself would
// ---------------------------------------------------------------------------------------------------
__global__ void rotary_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                    const int* __restrict__ position_ids, float2* __restrict__ out, int n_tokens, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const long total = (long)n_tokens * half;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / half), p = (int)(i - (long)t * half);
    float sn, cs;
    sincosf((float)(position_ids ? position_ids[t] : positions[t]) * inv_freq[p], &sn, &cs);
    out[i] = make_float2(sn, cs);
  }
}

FMS_API int fms_rotary_table(const float* inv_freq, const int* positions, const int* position_ids, void* out, int n_tokens,
                             int half, cudaStream_t stream) {
  if (n_tokens <= 0 || half <= 0) return 0;
  const long total = (long)n_tokens * half;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  fms_launch(rotary_table_kernel, dim3(blocks), dim3(256), 0, stream, inv_freq, positions, position_ids, (float2*)out,
             n_tokens, half);
  return fms_launch_status("rotary_table");
}

// ---------------------------------------------------------------------------------------------------
// start of a decode step: every sequence's new token sits at its current length, which then grows by one; the
// position its encoding sees is that place plus the offset at which the sequence started (offsets null: none)
// ---------------------------------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ positions, int* __restrict__ lengths,
                                      const int* __restrict__ offsets, int* __restrict__ position_ids,
                                      const int* __restrict__ slots, int spare_slot, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    // a row that only fills the step up to a size with a captured graph sits in the cache's spare slot and stays at
    // its first position, whatever the array held
    const int len = (slots != nullptr && slots[i] == spare_slot) ? 0 : lengths[i];
    positions[i] = len;
    lengths[i] = len + 1;
    if (offsets != nullptr) position_ids[i] = len + offsets[i];
  }
}

// slots, spare_slot: rows whose slot is spare_slot restart at position 0 every step (slots null: no such rows)
FMS_API int fms_decode_advance(int* positions, int* lengths, const int* offsets, int* position_ids, const int* slots,
                               int spare_slot, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((offsets == nullptr) != (position_ids == nullptr)) return fms_fail("decode_advance: offsets without position_ids");
  fms_launch(decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, positions, lengths, offsets, position_ids,
             slots, spare_slot, n);
  return fms_launch_status("decode_advance");
}

// ---------------------------------------------------------------------------------------------------
// norm after the sum (a layer whose norm follows the residual sum instead of preceding the sublayer):
//   x = alpha * residual[r] + sa * da[r] (+ sb * db[r]);  y = x / sqrt(mean(x^2) + eps) * gain
//   residual[r] = y (float32, in place);  copy[r] = y in the compute dtype, where a copy is asked for
// The sublayer's output may come as two parts with a factor each (two mixers side by side).  One block per row.
// No pointer is declared __restrict__ and nothing is read ahead of griddepcontrol.wait.
// ---------------------------------------------------------------------------------------------------
template <typename T, typename TG>
__global__ void scaled_add_rmsnorm_kernel(float* residual, float alpha, const T* da, float sa, const T* db, float sb,
                                          const TG* gain, float eps, T* copy, int dim) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * dim;
  float* res = residual + base;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float x = alpha * res[d];
    if (da) x = fmaf(sa, to_f32(da[base + d]), x);
    if (db) x = fmaf(sb, to_f32(db[base + d]), x);
    res[d] = x;
    ss += x * x;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float y = res[d] * inv * to_f32(gain[d]);  // this thread's own earlier store
    res[d] = y;
    if (copy) copy[base + d] = from_f32<T>(y);
  }
}

FMS_API int fms_scaled_add_rmsnorm(float* residual, float alpha, const void* da, float sa, const void* db, float sb,
                                   const void* gain, int gain_dtype, float eps, void* copy, int dtype, int n_rows, int dim,
                                   cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return fms_fail("scaled_add_rmsnorm: dim %d", dim);
  const int threads = dim >= 4096 ? 1024 : (dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128));
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(scaled_add_rmsnorm_kernel<T, TG>, dim3(n_rows), dim3(threads), 0, stream, residual, alpha,
                                (const T*)da, sa, (const T*)db, sb, (const TG*)gain, eps, (T*)copy, dim)));
  return fms_launch_status("scaled_add_rmsnorm");
}

// four consecutive values at once (the pointer aligned to four values)
__device__ __forceinline__ void ldv4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ldv4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void stv4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void stv4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const uint32_t*>(&a);
  t.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// float32 rows in the compute dtype (the stream as a sublayer's input where nothing else has made that copy)
template <typename T>
__global__ void cast_rows_kernel(const float* x, T* out, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    float v[4];
    ldv4(x + i, v);
    stv4(out + i, v);
  } else {
    for (size_t k = i; k < n; ++k) out[k] = from_f32<T>(x[k]);
  }
}

FMS_API int fms_cast_rows(const float* x, void* out, int dtype, long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((uintptr_t)x % 16 || (uintptr_t)out % 16) return fms_fail("cast_rows: rows that do not start on 16 bytes");
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(cast_rows_kernel<T>, dim3((unsigned)((n + 1023) / 1024)), dim3(256), 0, stream, x,
                                          (T*)out, (size_t)n));
  return fms_launch_status("cast_rows");
}

// ---------------------------------------------------------------------------------------------------
// norm in groups, for layers whose sublayers run side by side on the same stream:
//   x = residual[r] + s0 d0[r] + s1 d1[r] + s2 d2[r] + s3 d3[r]        (the parts that are given; float32)
//   residual[r] = x                                                     (not with `rows`: then row rows[i] is read)
//   the row in `groups` equal consecutive runs, each run y = x / sqrt(mean(x^2 over the run) + eps)
//   out1 = y * gain1, out2 = y * gain2 (where asked for): two norms of the same stream share their statistics
// A warp per (row, run), or a block per (row, run) for runs of 1,024 values and more; four values a thread where the
// run's size and the addresses allow.  The sums of a run are taken in the same order whatever else the step holds.
// ---------------------------------------------------------------------------------------------------
struct NormParts {
  const void* d[4];
  float s[4];
};

template <typename T, int VEC, bool WHOLE_BLOCK>
__global__ void parts_group_rmsnorm_kernel(float* residual, NormParts parts, const float* gain1, const float* gain2, float eps,
                                           int groups, T* out1, T* out2, const int* rows, int n_rows, int dim, int n_res) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int lane_n = WHOLE_BLOCK ? blockDim.x : 32;
  const int lane = WHOLE_BLOCK ? threadIdx.x : (threadIdx.x & 31);
  const long item = WHOLE_BLOCK ? (long)blockIdx.x : (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)n_rows * groups) return;  // a warp (or the block) as a whole
  const int r = (int)(item / groups), grp = (int)(item - (long)r * groups);
  const int gs = dim / groups;
  int src = r;
  if (rows) {
    src = __ldcg(rows + r);
    if (!FMS_IN(src, n_res)) return;
  }
  const size_t at = (size_t)src * dim + (size_t)grp * gs, out_at = (size_t)r * dim + (size_t)grp * gs;
  float* res = residual + at;
  const bool write_res = rows == nullptr;
  auto summed = [&](int e, float (&x)[VEC]) {
    if constexpr (VEC == 4) {
      ldv4(res + e, x);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (parts.d[k]) {
          float v[4];
          ldv4((const T*)parts.d[k] + at + e, v);
#pragma unroll
          for (int j = 0; j < 4; ++j) x[j] = fmaf(parts.s[k], v[j], x[j]);
        }
      }
    } else {
      x[0] = res[e];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (parts.d[k]) x[0] = fmaf(parts.s[k], to_f32(((const T*)parts.d[k])[at + e]), x[0]);
    }
  };
  float ss = 0.f;
  for (int e = lane * VEC; e < gs; e += lane_n * VEC) {
    float x[VEC];
    summed(e, x);
#pragma unroll
    for (int j = 0; j < VEC; ++j) ss += x[j] * x[j];
    if (write_res) {
      if constexpr (VEC == 4) stv4(res + e, x);
      else res[e] = x[0];
    }
  }
  const float total = WHOLE_BLOCK ? block_sum(ss, scratch) : warp_sum(ss);
  const float inv = 1.f / sqrtf(total / (float)gs + eps);
  for (int e = lane * VEC; e < gs; e += lane_n * VEC) {
    float x[VEC];
    if (write_res) {  // this thread's own earlier store
      if constexpr (VEC == 4) ldv4(res + e, x);
      else x[0] = res[e];
    } else {
      summed(e, x);
    }
    float y[VEC];
    if (out1) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) y[j] = x[j] * inv * gain1[grp * gs + e + j];
      if constexpr (VEC == 4) stv4(out1 + out_at + e, y);
      else out1[out_at + e] = from_f32<T>(y[0]);
    }
    if (out2) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) y[j] = x[j] * inv * gain2[grp * gs + e + j];
      if constexpr (VEC == 4) stv4(out2 + out_at + e, y);
      else out2[out_at + e] = from_f32<T>(y[0]);
    }
  }
}

FMS_API int fms_parts_group_rmsnorm(float* residual, const void* d0, float s0, const void* d1, float s1, const void* d2,
                                    float s2, const void* d3, float s3, const float* gain1, const float* gain2, float eps,
                                    int groups, void* out1, void* out2, int dtype, const int* rows, int n_rows, int dim,
                                    int n_res, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0 || groups <= 0 || dim % groups) return fms_fail("parts_group_rmsnorm: a row of %d values in %d runs", dim, groups);
  if ((out1 && !gain1) || (out2 && !gain2)) return fms_fail("parts_group_rmsnorm: an output without its gain");
  NormParts parts{{d0, d1, d2, d3}, {s0, s1, s2, s3}};
  const int gs = dim / groups;
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  bool four = gs % 4 == 0 && (uintptr_t)residual % 16 == 0 && (uintptr_t)out1 % (4 * item) == 0 && (uintptr_t)out2 % (4 * item) == 0;
  for (int k = 0; k < 4; ++k) four = four && (uintptr_t)parts.d[k] % (4 * item) == 0;
  const long items = (long)n_rows * groups;
  const bool whole = gs >= 1024;
  const dim3 grid((unsigned)(whole ? items : (items + 3) / 4)), block(whole ? (gs >= 4096 ? 512 : 256) : 128);
#define FMS_GROUP_NORM(VEC, WHOLE)                                                                                      \
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(parts_group_rmsnorm_kernel<T, VEC, WHOLE>, grid, block, 0, stream, residual, parts, \
                                          gain1, gain2, eps, groups, (T*)out1, (T*)out2, rows, n_rows, dim, n_res))
  if (four && whole) FMS_GROUP_NORM(4, true);
  else if (four) FMS_GROUP_NORM(4, false);
  else if (whole) FMS_GROUP_NORM(1, true);
  else FMS_GROUP_NORM(1, false);
#undef FMS_GROUP_NORM
  return fms_launch_status("parts_group_rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// queries, keys and values of a step on their way into attention, for heads whose first `rot` values are rotated,
// whose queries and keys may be divided by their root mean square afterwards, and whose value size may differ from
// the key size:
//   proj[t] = [q: nheads x dim | k: kvheads x dim | v: kvheads x vdim | ...]   (row stride `stride`)
//   q, k: pairs (2i, 2i+1), i < rot / 2, rotated by position * inv_freq[i]; the other values pass
//         (`halves`: the pairs are (i, i + rot / 2) instead; `rot_mult` multiplies the sines and cosines, 1 for a
//         plain rotation: stretched frequencies come with such a constant)
//   q, k: x / sqrt(mean(x^2) + eps) over the head's dim values, where qk_norm is set (no gain)
//         (`norm_first`: the norm comes before the rotation, times q_gain / k_gain [dim] where those are given)
//   `v_from_k`: there are no value columns; the value is the key as projected, before norm and rotation
//   q -> q_out[t, head, 0..pad) ; k, v -> the cache row of the token's slot and place, each `pad` wide:
//   values beyond dim (vdim) are zeros, so that kernels built for one head size `pad` serve both
// A warp per (token, head), four a block; float32 arithmetic.
// ---------------------------------------------------------------------------------------------------
constexpr int PREP_MAX_PAIRS = 256;

template <typename T>
__global__ void qk_prepare_store_kernel(const T* proj, int stride, T* q_out, const float* inv_freq, int rot,
                                        float rot_mult, int qk_norm, float eps, const float* q_gain, const float* k_gain, int norm_first,
                                        int halves, int v_from_k, const int* positions, const int* position_ids,
                                        const int* token_seq, const int* slots, T* k_cache, T* v_cache, const int* table,
                                        int table_stride, int block_tokens, int nheads, int kvheads, int dim, int vdim,
                                        int pad, int write_cache, int* error_flag, int n_seqs, int table_rows,
                                        int pool_blocks) {
  __shared__ float2 sc[PREP_MAX_PAIRS];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = __ldcg(positions + t);
  const int pid = position_ids ? __ldcg(position_ids + t) : pos;
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    float s, c;
    sincosf((float)pid * inv_freq[i], &s, &c);
    sc[i] = make_float2(s * rot_mult, c * rot_mult);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);  // a warp per head
  const T* row = proj + (size_t)t * stride;
  T* krow = nullptr;
  T* vrow = nullptr;
  if (write_cache) {
    const int seq = token_seq[t];
    if (FMS_IN(seq, n_seqs)) {
      const int slot = __ldcg(slots + seq);
      if (FMS_IN(slot, table_rows) && FMS_IN(pos / block_tokens, table_stride)) {
        const int blk = table[(size_t)slot * table_stride + pos / block_tokens];
        if (blk < 0) {
          if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
        } else if (FMS_IN(blk, pool_blocks)) {
          const size_t at = ((size_t)blk * kvheads * block_tokens + (pos % block_tokens)) * pad;
          krow = k_cache + at;  // head h of this token: + h * block_tokens * pad
          vrow = v_cache + at;
        }
      }
    }
  }
  if (item < nheads + 2 * kvheads) {
    if (item >= nheads + kvheads) {  // a value head: copied and padded
      const int h = item - nheads - kvheads;
      if (vrow == nullptr) return;
      const T* src = v_from_k ? row + (size_t)(nheads + h) * dim : row + (size_t)(nheads + kvheads) * dim + (size_t)h * vdim;
      T* dst = vrow + (size_t)h * block_tokens * pad;
      for (int e = lane; e < pad; e += 32) dst[e] = e < vdim ? src[e] : from_f32<T>(0.f);
      return;
    }
    const bool is_q = item < nheads;
    const T* src = row + (size_t)item * dim;  // q heads, then k heads, all `dim` wide
    T* dst = is_q ? q_out + ((size_t)t * nheads + item) * pad
                  : (krow ? krow + (size_t)(item - nheads) * block_tokens * pad : nullptr);
    if (dst == nullptr) return;
    const int half = rot / 2;
    if (norm_first) {
      // the norm (with its gain, where there is one) comes first and the rotation turns the normed values
      const float* gain = is_q ? q_gain : k_gain;
      float ss = 0.f;
      for (int e = lane; e < dim; e += 32) {
        const float x = to_f32(src[e]);
        ss += x * x;
      }
      const float inv = qk_norm ? 1.f / sqrtf(warp_sum(ss) / (float)dim + eps) : 1.f;
      for (int i = lane; i < half; i += 32) {
        const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
        const float x0 = to_f32(src[a]) * inv * (gain ? gain[a] : 1.f), x1 = to_f32(src[b]) * inv * (gain ? gain[b] : 1.f);
        dst[a] = from_f32<T>(sc[i].y * x0 - sc[i].x * x1);
        dst[b] = from_f32<T>(sc[i].y * x1 + sc[i].x * x0);
      }
      for (int e = rot + lane; e < pad; e += 32)
        dst[e] = from_f32<T>(e < dim ? to_f32(src[e]) * inv * (gain ? gain[e] : 1.f) : 0.f);
      return;
    }
    float ss = 0.f;
    for (int i = lane; i < half; i += 32) {
      const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
      const float x0 = to_f32(src[a]), x1 = to_f32(src[b]);
      const float r0 = sc[i].y * x0 - sc[i].x * x1, r1 = sc[i].y * x1 + sc[i].x * x0;
      ss += r0 * r0 + r1 * r1;
    }
    for (int e = rot + lane; e < dim; e += 32) {
      const float x = to_f32(src[e]);
      ss += x * x;
    }
    const float inv = qk_norm ? 1.f / sqrtf(warp_sum(ss) / (float)dim + eps) : 1.f;
    for (int i = lane; i < half; i += 32) {
      const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
      const float x0 = to_f32(src[a]), x1 = to_f32(src[b]);
      dst[a] = from_f32<T>((sc[i].y * x0 - sc[i].x * x1) * inv);
      dst[b] = from_f32<T>((sc[i].y * x1 + sc[i].x * x0) * inv);
    }
    for (int e = rot + lane; e < pad; e += 32) dst[e] = from_f32<T>(e < dim ? to_f32(src[e]) * inv : 0.f);
  }
}

FMS_API int fms_qk_prepare_store(const void* proj, int dtype, int stride, void* q_out, const float* inv_freq, int rot,
                                 float rot_mult, int qk_norm, float eps, const float* q_gain, const float* k_gain, int norm_first,
                                 int halves, int v_from_k, const int* positions, const int* position_ids,
                                 const int* token_seq, const int* slots, void* k_cache, void* v_cache, const int* table,
                                 int table_stride, int block_tokens, int n_tokens, int nheads, int kvheads, int dim,
                                 int vdim, int pad, int write_cache, int* error_flag, int n_seqs, int table_rows,
                                 int pool_blocks, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rot < 0 || rot % 2 || rot > dim || rot / 2 > PREP_MAX_PAIRS || (rot > 0 && inv_freq == nullptr))
    return fms_fail("qk_prepare_store: %d rotated values of %d", rot, dim);
  if (dim <= 0 || vdim <= 0 || pad < dim || pad < vdim) return fms_fail("qk_prepare_store: dim %d, vdim %d, pad %d", dim, vdim, pad);
  if (v_from_k && vdim != dim) return fms_fail("qk_prepare_store: values that are the keys have the keys' size, not %d for %d", vdim, dim);
  if ((q_gain || k_gain) && !norm_first) return fms_fail("qk_prepare_store: gains belong to the norm that comes before the rotation");
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(qk_prepare_store_kernel<T>, dim3(n_tokens, (nheads + 2 * kvheads + 3) / 4), dim3(128), 0, stream,
                                (const T*)proj, stride,
                                (T*)q_out, inv_freq, rot, rot_mult, qk_norm, eps, q_gain, k_gain, norm_first, halves, v_from_k,
                                positions, position_ids, token_seq, slots,
                                (T*)k_cache, (T*)v_cache, table, table_stride, block_tokens, nheads, kvheads, dim, vdim, pad,
                                write_cache, error_flag, n_seqs, table_rows, pool_blocks));
  return fms_launch_status("qk_prepare_store");
}

// ---------------------------------------------------------------------------------------------------
// gate on the heads' results: out[t, h * vdim + e] = factor * o[t, h * pad + e] * sigmoid(gate[t, h * vdim + e]),
// e < vdim; o has rows of nheads * pad, gate is a run of columns of a wider matrix (row stride gate_stride)
// `per_head`: one gate a head, sigmoid(gate[t, h]), instead of one a value
// ---------------------------------------------------------------------------------------------------
// VEC values a thread (4 where the sizes and addresses allow accesses of 4 values, else 1)
template <typename T, int VEC>
__global__ void sigmoid_gate_kernel(const T* o, const T* gate, int gate_stride, T* out, int nheads, int vdim, int pad,
                                    float factor, int per_head, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= total) return;
  const int width = nheads * vdim;
  const size_t t = i / width;
  const int c = (int)(i - t * width), h = c / vdim, e = c - h * vdim;
  if constexpr (VEC == 4) {
    float v[4], g[4];
    ldv4(o + (t * nheads + h) * pad + e, v);
    if (gate && per_head) g[0] = g[1] = g[2] = g[3] = to_f32(gate[t * gate_stride + h]);
    else if (gate) ldv4(gate + t * gate_stride + c, g);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = v[k] * factor * (gate ? 1.f / (1.f + expf(-g[k])) : 1.f);
    stv4(out + i, v);
  } else {
    float v = to_f32(o[(t * nheads + h) * pad + e]) * factor;
    if (gate) v *= 1.f / (1.f + expf(-to_f32(gate[t * gate_stride + (per_head ? h : c)])));
    out[i] = from_f32<T>(v);
  }
}

FMS_API int fms_sigmoid_gate(const void* o, const void* gate, int gate_stride, void* out, int dtype, int n_tokens,
                             int nheads, int vdim, int pad, float factor, int per_head, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const size_t total = (size_t)n_tokens * nheads * vdim;
  const size_t item = dtype == FMS_BF16 ? 2 : 4;
  const bool four = vdim % 4 == 0 && pad % 4 == 0 && (uintptr_t)o % (4 * item) == 0 && (uintptr_t)out % (4 * item) == 0 &&
                    (gate == nullptr || per_head || (gate_stride % 4 == 0 && (uintptr_t)gate % (4 * item) == 0));
  if (four) {
    FMS_DISPATCH_DTYPE(dtype, T, fms_launch(sigmoid_gate_kernel<T, 4>, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0,
                                            stream, (const T*)o, (const T*)gate, gate_stride, (T*)out, nheads, vdim, pad,
                                            factor, per_head, total));
  } else {
    FMS_DISPATCH_DTYPE(dtype, T, fms_launch(sigmoid_gate_kernel<T, 1>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                            (const T*)o, (const T*)gate, gate_stride, (T*)out, nheads, vdim, pad, factor, per_head, total));
  }
  return fms_launch_status("sigmoid_gate");
}
