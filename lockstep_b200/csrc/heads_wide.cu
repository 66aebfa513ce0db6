// Finishing a q/k/v projection whose heads the per-head kernel does not take:
//   - an RMSNorm over the whole query projection and one over the whole key projection
//     (gains of those sizes), or one per head, or none;
//   - key heads of size d and value heads of size dv that need not be equal;
//   - a layer that projects queries only (it reads another layer's keys and values);
//   - biases of the three projections, added here (in float32) rather than in the product;
//   - a query temperature: the query of position p times 1 + coef ln(floor((p + 1) / every) + 1).
// Queries go to q_out [tokens, nq * D], keys and values into the cache pages
// [num_pages, 2, nkv, page_size, D]; D >= max(d, dv) is the one head size the attention
// kernels then work with, and the elements past d (dv) are written as zeros: a zero in a
// query or key adds nothing to a score, a zero value column gives a zero output column.
// One block per token.  Sums of squares are taken in float32 in a fixed order (a thread's
// elements ascending, lanes by xor-tree, warps ascending), so a token's bits do not depend
// on the batch.  Rotation: the halves layout on the first rot_dim elements of each head,
// products and sums rounded one by one as in rope.cuh.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

struct WideArgs {
  const void* qkv;          // [tokens, ld]: q (nq*d), then k (nkv*d) and v (nkv*dv) if has_kv
  void* q_out;
  void* pages;
  const void* q_gain;       // scope 2: [nq*d]; scope 1: [d]; null: no norm
  const void* k_gain;
  const float* cos_table;   // [max_positions, rot_dim / 2]
  const float* sin_table;
  const int* positions;
  const int* token_req;
  const int* block_table;
  int64_t ld;
  int gain_bf16, table_stride, tokens, nq, nkv, d, dv, D, rot_dim, page_size, num_pages, max_positions;
  int scope;                // 0 none, 1 per head, 2 whole projection
  int has_kv, write_cache;
  float eps;
  const void* bias;         // null, or [ld]: the biases of q, k, v in the order of the projection's columns
  int bias_bf16;
  float temp_coef;          // query temperature (0: none)
  int temp_every;
};

__device__ __forceinline__ float gain_at(const void* g, int bf16, int i) {
  return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])
              : reinterpret_cast<const float*>(g)[i];
}

// element i of a projection's row (at column `col0` of the whole row), with its bias
template <typename T>
__device__ __forceinline__ float biased_at(const WideArgs& a, const T* src, int col0, int i) {
  const float v = ls_to_float<T>(src[i]);
  return a.bias != nullptr ? v + gain_at(a.bias, a.bias_bf16, col0 + i) : v;
}

// sum of squares of src[0 .. n) by the whole block, fixed order
template <typename T>
__device__ float block_sumsq(const WideArgs& a, const T* src, int col0, int n, float* scratch) {
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const float v = biased_at<T>(a, src, col0, i);
    ss = fmaf(v, v, ss);
  }
  return ls_block_sum(ss, scratch);
}

// One projection (q or k) of one token: heads of size d at src, normed, rotated, written as
// heads of size D at dst(head) (the padding as zeros).
template <typename T, typename Dst>
__device__ void finish_heads(const WideArgs& a, const T* src, int col0, int heads, const void* gain, float rstd_whole,
                             const float* cs, const float* sn, float* head_rstd, float factor, Dst dst) {
  const int d = a.d, D = a.D, half = a.rot_dim >> 1;
  if (a.scope == 1 && gain != nullptr) {
    // per-head sums: a warp per head, lanes strided, xor-tree
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int h = warp; h < heads; h += THREADS / 32) {
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) {
        const float v = biased_at<T>(a, src, col0, h * d + i);
        ss = fmaf(v, v, ss);
      }
      ss = ls_warp_sum(ss);
      if (lane == 0) head_rstd[h] = 1.0f / sqrtf(ss / (float)d + a.eps);
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < heads * D; e += THREADS) {
    const int h = e / D, i = e - h * D;
    float out = 0.f;
    if (i < d) {
      auto normed = [&](int j) {
        float v = biased_at<T>(a, src, col0, h * d + j);
        if (gain != nullptr) {
          v = __fmul_rn(v, a.scope == 2 ? rstd_whole : head_rstd[h]);
          v = __fmul_rn(v, gain_at(gain, a.gain_bf16, a.scope == 2 ? h * d + j : j));
        }
        return v;
      };
      if (i < a.rot_dim) {
        if (i < half) {
          const float lo = normed(i), hi = normed(i + half);
          out = __fsub_rn(__fmul_rn(lo, cs[i]), __fmul_rn(hi, sn[i]));
        } else {
          const float lo = normed(i - half), hi = normed(i);
          out = __fadd_rn(__fmul_rn(hi, cs[i - half]), __fmul_rn(lo, sn[i - half]));
        }
      } else {
        out = normed(i);
      }
      if (factor != 1.0f) out = __fmul_rn(out, factor);
    }
    dst(h, i, out);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) qkv_finish_kernel(WideArgs a, int* err) {
  __shared__ float scratch[32];
  __shared__ float head_rstd[256];
  ls_dependency_sync();
  const int t = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(a.qkv) + (int64_t)t * a.ld;
  const int pos = a.positions[t];
  const int half = a.rot_dim >> 1;
  if (half > 0 && (pos < 0 || pos >= a.max_positions)) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_POSITION_RANGE, t);
    return;
  }
  const float* cs = a.cos_table + (int64_t)pos * half;
  const float* sn = a.sin_table + (int64_t)pos * half;

  // queries
  float rstd = 1.f;
  if (a.scope == 2 && a.q_gain != nullptr)
    rstd = 1.0f / sqrtf(block_sumsq<T>(a, row, 0, a.nq * a.d, scratch) / (float)(a.nq * a.d) + a.eps);
  T* q_dst = reinterpret_cast<T*>(a.q_out) + (int64_t)t * a.nq * a.D;
  const float temperature =
      a.temp_coef != 0.f ? 1.0f + a.temp_coef * logf((float)((pos + 1) / a.temp_every + 1)) : 1.0f;
  finish_heads<T>(a, row, 0, a.nq, a.q_gain, rstd, cs, sn, head_rstd, temperature,
                  [&](int h, int i, float v) { q_dst[h * a.D + i] = ls_from_float<T>(v); });
  if (!a.has_kv || !a.write_cache) return;

  // keys and values into the token's page
  const int req = a.token_req[t];
  const int page = a.block_table[(int64_t)req * a.table_stride + pos / a.page_size];
  if (page < 0 || page >= a.num_pages) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_PAGE_RANGE, t);
    return;
  }
  const int in_page = pos % a.page_size;
  T* pages = reinterpret_cast<T*>(a.pages);
  const T* k_src = row + a.nq * a.d;
  const T* v_src = k_src + a.nkv * a.d;
  float k_rstd = 1.f;
  if (a.scope == 2 && a.k_gain != nullptr) {
    __syncthreads();
    k_rstd = 1.0f / sqrtf(block_sumsq<T>(a, k_src, a.nq * a.d, a.nkv * a.d, scratch) / (float)(a.nkv * a.d) + a.eps);
  }
  __syncthreads();          // head_rstd is used again
  finish_heads<T>(a, k_src, a.nq * a.d, a.nkv, a.k_gain, k_rstd, cs, sn, head_rstd, 1.0f, [&](int h, int i, float v) {
    pages[((((int64_t)page * 2 + 0) * a.nkv + h) * a.page_size + in_page) * a.D + i] = ls_from_float<T>(v);
  });
  for (int e = threadIdx.x; e < a.nkv * a.D; e += THREADS) {
    const int h = e / a.D, i = e - h * a.D;
    pages[((((int64_t)page * 2 + 1) * a.nkv + h) * a.page_size + in_page) * a.D + i] =
        i < a.dv ? ls_from_float<T>(biased_at<T>(a, v_src, (a.nq + a.nkv) * a.d, h * a.dv + i)) : ls_from_float<T>(0.f);
  }
}

}  // namespace

LS_API int ls_qkv_finish(const void* qkv, int64_t ld, void* q_out, void* pages, int dtype, const void* q_gain,
                         const void* k_gain, int gain_dtype, const float* cos_table, const float* sin_table,
                         const int* positions, const int* token_req, const int* block_table, int table_stride,
                         int tokens, int nq, int nkv, int d, int dv, int D, int rot_dim, int page_size,
                         int num_pages, int max_positions, float eps, int scope, int has_kv, int write_cache,
                         const void* bias, int bias_dtype, float temp_coef, int temp_every,
                         int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || D < d || D < dv || scope < 0 || scope > 2) return LS_E_SIZE;
  if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return LS_E_SIZE;
  if (scope == 1 && (nq > 256 || nkv > 256)) return LS_E_SIZE;
  if (gain_dtype != LS_F32 && gain_dtype != LS_BF16) return LS_E_DTYPE;
  if (write_cache && (pages == nullptr || page_size <= 0)) return LS_E_SIZE;
  if (temp_coef != 0.f && temp_every <= 0) return LS_E_SIZE;
  if (bias != nullptr && bias_dtype != LS_F32 && bias_dtype != LS_BF16) return LS_E_DTYPE;
  WideArgs a;
  a.bias = bias; a.bias_bf16 = bias_dtype == LS_BF16 ? 1 : 0; a.temp_coef = temp_coef; a.temp_every = temp_every > 0 ? temp_every : 1;
  a.qkv = qkv; a.q_out = q_out; a.pages = pages; a.q_gain = q_gain; a.k_gain = k_gain;
  a.cos_table = cos_table; a.sin_table = sin_table; a.positions = positions; a.token_req = token_req;
  a.block_table = block_table; a.ld = ld; a.gain_bf16 = gain_dtype == LS_BF16 ? 1 : 0;
  a.table_stride = table_stride; a.tokens = tokens; a.nq = nq; a.nkv = nkv; a.d = d; a.dv = dv; a.D = D;
  a.rot_dim = rot_dim; a.page_size = page_size > 0 ? page_size : 1; a.num_pages = num_pages;
  a.max_positions = max_positions; a.scope = (q_gain == nullptr && k_gain == nullptr) ? 0 : scope;
  a.has_kv = has_kv; a.write_cache = write_cache; a.eps = eps;
  LS_COUNT(LS_K_QKV_FINISH);
  cudaError_t e;
  if (dtype == LS_F32) e = ls_launch(qkv_finish_kernel<float>, dim3(tokens), dim3(THREADS), 0, stream, a, err);
  else if (dtype == LS_BF16) e = ls_launch(qkv_finish_kernel<__nv_bfloat16>, dim3(tokens), dim3(THREADS), 0, stream, a, err);
  else return LS_E_DTYPE;
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}
