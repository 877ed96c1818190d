// The gated delta rule and the short convolutions in front of it.
//
//   li_short_conv         y[t, c] = act(sum_m w[c, m] * x[t - (K-1-m), c]): a causal convolution over time per
//                         channel; inputs before the step come from the request's tail (its last K-1 inputs)
//   li_short_conv_update  moves every request's tail on by the step's inputs
//   li_gated_delta_rule   per request and head a state S [dim, vdim] in 32-bit; per token
//                             S *= g;  u = beta * (v - S^T k);  S += k u^T;  o = S^T q
//                         with q, k made unit vectors (q also times dim^-0.5), beta = sigmoid(raw),
//                         g = exp(-exp(A_log) * softplus(raw + dt_bias))
//
// The recurrence is a chain over the tokens of a sequence, but every column of S is a chain of its own:
// (S^T k)_j, u_j, the update of S[:, j] and o_j touch column j only.  So a block takes 32 columns of one head of
// one sequence, eight lanes share a column (each keeps dim/8 of its entries in registers for the whole step) and
// add up their parts of the two dot products with three shuffles.  Whole prompts, portions and single tokens run
// the same code from the state the step before left, in the same order, so the result does not depend on how a
// sequence was cut.  Tokens of padding (sequence -1) and sequences that bring no token touch nothing.
#include "common.cuh"

namespace li {

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ x, size_t x_stride, const T* __restrict__ taps,
                                  const T* __restrict__ tail, const int* __restrict__ seq_of_token,
                                  const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                                  T* __restrict__ out, int channels, int K, int act) {
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int seq = seq_of_token[t];
  if (seq < 0) {
    out[(size_t)t * channels + c] = from_float<T>(0.f);
    return;
  }
  const int j = t - query_start_loc[seq];   // index of the token among its sequence's tokens of this step
  const T* old = tail + (size_t)state_slots[seq] * (K - 1) * channels;
  float acc = 0.f;
  for (int m = 0; m < K; ++m) {
    const int back = K - 1 - m;
    const float in = back <= j ? to_float(x[(size_t)(t - back) * x_stride + c])
                               : to_float(old[(size_t)(K - 1 + j - back) * channels + c]);
    acc = fmaf(to_float(taps[(size_t)c * K + m]), in, acc);
  }
  if (act) acc = acc / (1.0f + expf(-acc));
  out[(size_t)t * channels + c] = from_float<T>(acc);
}

template <typename T>
__global__ void short_conv_update_kernel(const T* __restrict__ x, size_t x_stride, T* __restrict__ tail,
                                         const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                                         int channels, int K) {
  grid_dependency_wait();
  const int seq = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int begin = query_start_loc[seq], n = query_start_loc[seq + 1] - begin;
  if (n <= 0) return;
  const int keep = K - 1;
  T* mine = tail + (size_t)state_slots[seq] * keep * channels;
  // Entry i becomes the input at index n - keep + i of the step, or the old entry i + n where that lies before the
  // step; ascending i reads only entries that are not yet overwritten.
  for (int i = 0; i < keep; ++i) {
    const int li = n - keep + i;
    mine[(size_t)i * channels + c] = li >= 0 ? x[(size_t)(begin + li) * x_stride + c] : mine[(size_t)(i + n) * channels + c];
  }
}

__device__ __forceinline__ float sum_over_column_lanes(float v) {   // the eight lanes of a column: lane bits 2..4
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

template <typename T, int R>   // R: entries of a column that one lane keeps; dim <= 8 * R
struct DeltaToken {
  float q[R], k[R], v, beta_raw, decay_raw;
};

template <typename T, int R>
__device__ __forceinline__ void load_token(DeltaToken<T, R>& tok, const T* __restrict__ qkv, size_t row_width,
                                           const T* __restrict__ ab, size_t ab_stride, int t, int q_at, int k_at,
                                           int v_at, bool column_live, int first, int dim, int head, int heads) {
  const T* row = qkv + (size_t)t * row_width;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = first + r;
    tok.q[r] = i < dim ? to_float(row[q_at + i]) : 0.f;
    tok.k[r] = i < dim ? to_float(row[k_at + i]) : 0.f;
  }
  tok.v = column_live ? to_float(row[v_at]) : 0.f;
  tok.beta_raw = to_float(ab[(size_t)t * ab_stride + head]);
  tok.decay_raw = to_float(ab[(size_t)t * ab_stride + heads + head]);
}

template <typename T, int R>
__global__ void __launch_bounds__(256)
gated_delta_rule_kernel(const T* __restrict__ qkv, const T* __restrict__ ab, size_t ab_stride,
                        const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ state,
                        const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                        float* __restrict__ out, int heads, int kv_heads, int dim, int vdim) {
  grid_dependency_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int begin = query_start_loc[seq], end = query_start_loc[seq + 1];
  if (end <= begin) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane >> 2;                                   // which eighth of the column
  const int column = blockIdx.x * 32 + warp * 4 + (lane & 3);
  const bool live = column < vdim;
  const int first = part * R;
  const int qk_width = kv_heads * dim;
  const size_t row_width = 2 * (size_t)qk_width + (size_t)heads * vdim;
  const int kv_head = head / (heads / kv_heads);
  const int q_at = kv_head * dim, k_at = qk_width + kv_head * dim, v_at = 2 * qk_width + head * vdim + column;
  float* mine = state + (((size_t)state_slots[seq] * heads + head) * dim) * vdim + column;

  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = (live && first + r < dim) ? mine[(size_t)(first + r) * vdim] : 0.f;
  const float rate = expf(a_log[head]), bias = dt_bias[head];
  const float q_scale = 1.0f / sqrtf((float)dim);

  DeltaToken<T, R> cur, next;
  load_token<T, R>(cur, qkv, row_width, ab, ab_stride, begin, q_at, k_at, v_at, live, first, dim, head, heads);
  for (int t = begin; t < end; ++t) {
    if (t + 1 < end)
      load_token<T, R>(next, qkv, row_width, ab, ab_stride, t + 1, q_at, k_at, v_at, live, first, dim, head, heads);
    float qq = 0.f, kk = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      qq = fmaf(cur.q[r], cur.q[r], qq);
      kk = fmaf(cur.k[r], cur.k[r], kk);
    }
    qq = sum_over_column_lanes(qq);
    kk = sum_over_column_lanes(kk);
    const float q_inv = q_scale / sqrtf(qq + 1e-6f), k_inv = 1.0f / sqrtf(kk + 1e-6f);
    const float beta = 1.0f / (1.0f + expf(-cur.beta_raw));
    const float z = cur.decay_raw + bias;
    const float soft = z > 20.f ? z : log1pf(expf(z));
    const float g = expf(-rate * soft);
    float dot = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      cur.k[r] *= k_inv;
      S[r] *= g;
      dot = fmaf(S[r], cur.k[r], dot);
    }
    dot = sum_over_column_lanes(dot);
    const float u = beta * (cur.v - dot);
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] = fmaf(cur.k[r], u, S[r]);
      o = fmaf(S[r], cur.q[r] * q_inv, o);
    }
    o = sum_over_column_lanes(o);
    if (live && part == 0) out[(size_t)t * heads * vdim + (size_t)head * vdim + column] = o;
    cur = next;
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (live && first + r < dim) mine[(size_t)(first + r) * vdim] = S[r];
}

template <typename T>
int launch_delta(int dim, dim3 grid, cudaStream_t stream, const T* qkv, const T* ab, size_t ab_stride, const float* a_log,
                 const float* dt_bias, float* state, const int* qsl, const int* slots, float* out, int heads, int kv_heads,
                 int vdim, int tokens) {
#define LI_DELTA(R)                                                                                                  \
  return (int)launch_pdl(tokens, gated_delta_rule_kernel<T, R>, grid, dim3(256), 0, stream, qkv, ab, ab_stride, a_log, \
                         dt_bias, state, qsl, slots, out, heads, kv_heads, dim, vdim)
  if (dim <= 32) LI_DELTA(4);
  if (dim <= 64) LI_DELTA(8);
  if (dim <= 128) LI_DELTA(16);
  if (dim <= 256) LI_DELTA(32);
#undef LI_DELTA
  return LI_ERR_UNSUPPORTED;
}

}  // namespace li

using namespace li;

LI_EXPORT int li_short_conv(int dtype, const void* x, size_t x_stride, const void* taps, const void* tail,
                            const int* seq_of_token, const int* query_start_loc, const int* state_slots, void* out,
                            int tokens, int channels, int K, int act, cudaStream_t stream) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (K < 1 || K > kMaxTaps || (K > 1 && tail == nullptr) || (channels + 127) / 128 > 65535) return LI_ERR_UNSUPPORTED;
  const dim3 grid(tokens, (channels + 127) / 128);
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, short_conv_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, x_stride,
                           (const float*)taps, (const float*)tail, seq_of_token, query_start_loc, state_slots,
                           (float*)out, channels, K, act);
  return (int)launch_pdl(tokens, short_conv_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)x, x_stride,
                         (const bf16*)taps, (const bf16*)tail, seq_of_token, query_start_loc, state_slots, (bf16*)out,
                         channels, K, act);
}

LI_EXPORT int li_short_conv_update(int dtype, const void* x, size_t x_stride, void* tail, const int* query_start_loc,
                                   const int* state_slots, int num_seqs, int channels, int K, cudaStream_t stream) {
  if (num_seqs <= 0 || channels <= 0 || K <= 1) return 0;
  if (K > kMaxTaps || num_seqs > 65535) return LI_ERR_UNSUPPORTED;
  const dim3 grid((channels + 127) / 128, num_seqs);
  if (dtype == kFloat32)
    return (int)launch_pdl(num_seqs, short_conv_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)x,
                           x_stride, (float*)tail, query_start_loc, state_slots, channels, K);
  return (int)launch_pdl(num_seqs, short_conv_update_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)x, x_stride,
                         (bf16*)tail, query_start_loc, state_slots, channels, K);
}

// qkv [tokens, 2 * kv_heads * dim + heads * vdim]; ab [tokens, >= 2 * heads] with `ab_stride` elements a row; state
// [slots, heads, dim, vdim]; out [tokens, heads * vdim], both float.
LI_EXPORT int li_gated_delta_rule(int dtype, const void* qkv, const void* ab, size_t ab_stride, int tokens, int num_seqs,
                                  const float* a_log, const float* dt_bias, float* state, const int* query_start_loc,
                                  const int* state_slots, float* out, int heads, int kv_heads, int dim, int vdim, int,
                                  int, cudaStream_t stream) {
  if (tokens <= 0 || num_seqs <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || vdim < 1 || heads > 65535 || num_seqs > 65535)
    return LI_ERR_UNSUPPORTED;
  const dim3 grid((vdim + 31) / 32, heads, num_seqs);
  if (dtype == kFloat32)
    return launch_delta<float>(dim, grid, stream, (const float*)qkv, (const float*)ab, ab_stride, a_log, dt_bias, state,
                               query_start_loc, state_slots, out, heads, kv_heads, vdim, tokens);
  return launch_delta<bf16>(dim, grid, stream, (const bf16*)qkv, (const bf16*)ab, ab_stride, a_log, dt_bias, state,
                            query_start_loc, state_slots, out, heads, kv_heads, vdim, tokens);
}
