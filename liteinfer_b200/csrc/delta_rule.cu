// The gated delta rule and the short convolutions in front of it.
//
//   li_short_conv         y[t, c] = act(sum_m w[m, c] * x[t - (K-1-m), c]): a causal convolution over time per
//                         channel (the taps tap by tap, [K, channels], so that neighbouring channels' weights are
//                         neighbours); inputs before the step come from the request's tail (its last K-1 inputs)
//   li_short_conv_update  moves every request's tail on by the step's inputs
//   li_gated_delta_rule   per request and head a state S [dim, vdim] in 32-bit (kept column by column); per token
//                             S *= g;  u = beta * (v - S^T k);  S += k u^T;  o = S^T q
//                         with q, k made unit vectors (q also times dim^-0.5), beta = sigmoid(raw),
//                         g = exp(-exp(A_log) * softplus(raw + dt_bias))
//
// The recurrence is a chain over the tokens of a sequence, but every column of S is a chain of its own:
// (S^T k)_j, u_j, the update of S[:, j] and o_j touch column j only.  So a block takes 32 columns of one head of
// one sequence, eight lanes share a column (each keeps dim/8 of its entries in registers for the whole step) and
// add up their parts of the two dot products with three shuffles.  What does not depend on the state (the unit
// norms, beta, the decay) is computed once per token and head by a kernel in front; the inputs of the next few
// tokens are in flight while one is computed.  Whole prompts, portions and single tokens run
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
    acc = fmaf(to_float(taps[(size_t)m * channels + c]), in, acc);
  }
  if (act) acc = acc / (1.0f + expf(-acc));
  out[(size_t)t * channels + c] = from_float<T>(acc);
}

// The same, a 16-byte vector of neighbouring channels a thread (channels and row strides multiples of the
// vector's length, 16-byte aligned pointers).
template <typename T>
__global__ void short_conv_vec_kernel(const T* __restrict__ x, size_t x_stride, const T* __restrict__ taps,
                                      const T* tail, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                                      T* __restrict__ out, int channels, int K, int act, T* move_tail) {
  // move_tail (only where every sequence of the step brings one token): the tail is also moved on here, by the
  // thread that has just read all of it for its channels (tail and move_tail are the same memory).
  constexpr int N = Vec16<T>::N;
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * N;
  if (c >= channels) return;
  const int seq = seq_of_token[t];
  Vec16<T> result;
  if (seq < 0) {
    grid_dependency_wait();
#pragma unroll
    for (int e = 0; e < N; ++e) result.set(e, 0.f);
    store16(out + (size_t)t * channels + c, result);
    return;
  }
  const int j = t - query_start_loc[seq];
  const T* old = tail + (size_t)state_slots[seq] * (K - 1) * channels;
  grid_dependency_wait();
  float acc[N];
#pragma unroll
  for (int e = 0; e < N; ++e) acc[e] = 0.f;
  for (int m = 0; m < K; ++m) {
    const int back = K - 1 - m;
    const Vec16<T> in = back <= j ? load16(x + (size_t)(t - back) * x_stride + c)
                                  : load16(old + (size_t)(K - 1 + j - back) * channels + c);
    float w[N], v[N];
    unpack16(load16(taps + (size_t)m * channels + c), w);
    unpack16(in, v);
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] = fmaf(w[e], v[e], acc[e]);
    // A step of one token (j = 0): tap m read tail entry m (or the token itself, m = K - 1), which becomes entry m - 1.
    if (move_tail != nullptr && m >= 1)
      store16(move_tail + ((size_t)state_slots[seq] * (K - 1) + (m - 1)) * channels + c, in);
  }
#pragma unroll
  for (int e = 0; e < N; ++e) {
    // bfloat16 results take the fast exponential and division (relative error about 1e-6, far inside the rounding).
    const float sig = sizeof(T) == 2 ? __fdividef(1.0f, 1.0f + __expf(-acc[e])) : 1.0f / (1.0f + expf(-acc[e]));
    result.set(e, act ? acc[e] * sig : acc[e]);
  }
  store16(out + (size_t)t * channels + c, result);
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

// What of a token does not depend on the state, once per (token, head) instead of once per column of S:
// units [tokens][kv_heads][2][dim] = (q dim^-0.5 / |q|, k / |k|) in float with |x| = sqrt(sum x^2 + 1e-6), and
// gates [tokens][heads][2] = (beta, g) = (sigmoid(raw_b), exp(-exp(A_log) * softplus(raw_a + dt_bias))).  One warp
// a (token, head or kv head).
template <typename T>
__global__ void delta_gates_kernel(const T* __restrict__ qkv, size_t row_width, const T* __restrict__ ab,
                                   size_t ab_stride, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ scales, float* __restrict__ gates, int tokens, int heads,
                                   int kv_heads, int dim) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int per_token = kv_heads + (heads + 31) / 32;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (size_t)tokens * per_token) return;
  const size_t t = item / per_token;
  const int what = (int)(item - t * per_token);
  if (what < kv_heads) {
    const T* q = qkv + t * row_width + (size_t)what * dim;
    const T* k = q + (size_t)kv_heads * dim;
    float qq = 0.f, kk = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float a = to_float(q[i]), b = to_float(k[i]);
      qq = fmaf(a, a, qq);
      kk = fmaf(b, b, kk);
    }
    qq = warp_sum(qq);
    kk = warp_sum(kk);
    const float q_inv = (1.0f / sqrtf((float)dim)) / sqrtf(qq + 1e-6f), k_inv = 1.0f / sqrtf(kk + 1e-6f);
    float* unit = scales + (t * kv_heads + what) * 2 * (size_t)dim;
    for (int i = lane; i < dim; i += 32) {
      unit[i] = to_float(q[i]) * q_inv;
      unit[dim + i] = to_float(k[i]) * k_inv;
    }
  } else {
    const int head = (what - kv_heads) * 32 + lane;
    if (head >= heads) return;
    const float raw_b = to_float(ab[t * ab_stride + head]), raw_a = to_float(ab[t * ab_stride + heads + head]);
    const float z = raw_a + dt_bias[head];
    const float soft = z > 20.f ? z : log1pf(expf(z));
    gates[(t * heads + head) * 2] = 1.0f / (1.0f + expf(-raw_b));
    gates[(t * heads + head) * 2 + 1] = expf(-expf(a_log[head]) * soft);
  }
}

// R values of T starting at p (R a multiple of 4; p aligned to 16 bytes when kVector) as floats.
template <typename T, int R, bool kVector>
__device__ __forceinline__ void load_slice(float (&dst)[R], const T* __restrict__ p, int live) {
  if (kVector) {
    constexpr int N = Vec16<T>::N;
#pragma unroll
    for (int c = 0; c < R / N; ++c) unpack16(load16(p + c * N), dst + c * N);
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) dst[r] = r < live ? to_float(p[r]) : 0.f;
  }
}

template <int R>
struct DeltaToken {   // what a lane needs of one token: its slices of q and k, its column's v, the head's scalars
  float q[R], k[R], v, q_inv, k_inv, beta, g;
};

// The state is kept column by column: state[slot][head][column][dim], so that a lane's slice of a column (R
// entries) is contiguous and a warp's four columns are 4 * dim * 4 bytes in a row.
// R: entries of a column that one lane keeps (dim <= 8 R).  kAhead: tokens whose inputs are in flight while one is
// computed (1 for steps of single tokens).  kVector: dim == 8 R and every row is 16-byte aligned.
template <typename T, int R, int kAhead, bool kVector>
__global__ void __launch_bounds__(256)
gated_delta_rule_kernel(const T* __restrict__ qkv, const float* __restrict__ scales, const float* __restrict__ gates,
                        float* __restrict__ state, const int* __restrict__ query_start_loc,
                        const int* __restrict__ state_slots, float* __restrict__ out, int heads, int kv_heads, int dim,
                        int vdim, const T* __restrict__ ab, size_t ab_stride, const float* __restrict__ a_log,
                        const float* __restrict__ dt_bias) {
  grid_dependency_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int begin = query_start_loc[seq], end = query_start_loc[seq + 1];
  if (end <= begin) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane >> 2;                                   // which eighth of the column
  const int column = blockIdx.x * 32 + warp * 4 + (lane & 3);
  const bool live = column < vdim;
  const int first = part * R;
  const int mine_dims = min(R, max(0, dim - first));            // entries of this lane's slice that exist
  const int qk_width = kv_heads * dim;
  const size_t row_width = 2 * (size_t)qk_width + (size_t)heads * vdim;
  const int kv_head = head / (heads / kv_heads);
  const size_t q_at = (size_t)kv_head * dim + first, k_at = (size_t)qk_width + q_at;
  const size_t v_at = 2 * (size_t)qk_width + (size_t)head * vdim + (live ? column : 0);
  float* mine = state + (((size_t)state_slots[seq] * heads + head) * vdim + (live ? column : 0)) * dim + first;

  float S[R];
  if (kVector) {
#pragma unroll
    for (int c = 0; c < R / 4; ++c) {
      const float4 v = live ? *reinterpret_cast<const float4*>(mine + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[c * 4] = v.x; S[c * 4 + 1] = v.y; S[c * 4 + 2] = v.z; S[c * 4 + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = (live && r < mine_dims) ? mine[r] : 0.f;
  }

  DeltaToken<R> ring[kAhead];
  auto fetch = [&](DeltaToken<R>& tok, int t) {
    const T* row = qkv + (size_t)t * row_width;
    tok.v = widen(row[v_at]);
    if (kAhead > 1) {
      // From the kernel in front: q and k as unit vectors in float, and the gates.
      const float* unit = scales + ((size_t)t * kv_heads + kv_head) * 2 * (size_t)dim + first;
      load_slice<float, R, kVector>(tok.q, unit, mine_dims);
      load_slice<float, R, kVector>(tok.k, unit + dim, mine_dims);
      const float2 ga = *reinterpret_cast<const float2*>(gates + ((size_t)t * heads + head) * 2);
      tok.q_inv = 1.f; tok.k_inv = 1.f; tok.beta = ga.x; tok.g = ga.y;
      return;
    }
    load_slice<T, R, kVector>(tok.q, row + q_at, mine_dims);
    load_slice<T, R, kVector>(tok.k, row + k_at, mine_dims);
    if (kAhead == 1) {
      // Steps of single tokens: no kernel in front; the block works out the token's scales and gates itself.
      float qq = 0.f, kk = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        qq = fmaf(tok.q[r], tok.q[r], qq);
        kk = fmaf(tok.k[r], tok.k[r], kk);
      }
      qq = sum_over_column_lanes(qq);
      kk = sum_over_column_lanes(kk);
      tok.q_inv = (1.0f / sqrtf((float)dim)) / sqrtf(qq + 1e-6f);
      tok.k_inv = 1.0f / sqrtf(kk + 1e-6f);
      const float raw_b = to_float(ab[(size_t)t * ab_stride + head]);
      const float z = to_float(ab[(size_t)t * ab_stride + heads + head]) + dt_bias[head];
      const float soft = z > 20.f ? z : log1pf(expf(z));
      tok.beta = 1.0f / (1.0f + expf(-raw_b));
      tok.g = expf(-expf(a_log[head]) * soft);
    }
  };
  // A token's read-out o = S^T q is not on the chain from token to token, only its S is: the lanes' parts of o
  // are added up together with the next token's parts of S^T k, so a token costs one round of shuffles.
  float o_parts = 0.f, o_scale = 0.f;
  int o_token = -1;
  auto step = [&](const DeltaToken<R>& tok, int t) {
    // With S' = g S:  (S'^T k)_j = g k_inv sum_i S_ij k_i;  S <- g S + k (k_inv u)^T;  o_j = q_inv sum_i S_ij q_i.
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      d0 = fmaf(S[r], tok.k[r], d0); d1 = fmaf(S[r + 1], tok.k[r + 1], d1);
      d2 = fmaf(S[r + 2], tok.k[r + 2], d2); d3 = fmaf(S[r + 3], tok.k[r + 3], d3);
    }
    float dsum = (d0 + d1) + (d2 + d3), osum = o_parts;
#pragma unroll
    for (int offset = 4; offset <= 16; offset <<= 1) {
      const float a = __shfl_xor_sync(0xffffffffu, dsum, offset), b = __shfl_xor_sync(0xffffffffu, osum, offset);
      dsum += a;
      osum += b;
    }
    if (o_token >= 0 && live && part == 0)
      out[(size_t)o_token * heads * vdim + (size_t)head * vdim + column] = osum * o_scale;
    const float dot = dsum * (tok.g * tok.k_inv);
    const float c = tok.beta * (tok.v - dot) * tok.k_inv;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      S[r] = fmaf(S[r], tok.g, tok.k[r] * c); S[r + 1] = fmaf(S[r + 1], tok.g, tok.k[r + 1] * c);
      S[r + 2] = fmaf(S[r + 2], tok.g, tok.k[r + 2] * c); S[r + 3] = fmaf(S[r + 3], tok.g, tok.k[r + 3] * c);
      o0 = fmaf(S[r], tok.q[r], o0); o1 = fmaf(S[r + 1], tok.q[r + 1], o1);
      o2 = fmaf(S[r + 2], tok.q[r + 2], o2); o3 = fmaf(S[r + 3], tok.q[r + 3], o3);
    }
    o_parts = (o0 + o1) + (o2 + o3);
    o_scale = tok.q_inv;
    o_token = t;
  };

  // Far ahead of the ring, the lines of a token's inputs are asked into the cache: warp w does it for the tokens
  // whose number is w modulo 8, one lane a 128-byte line (the unit vectors, then v, then the gates).
  constexpr int kFar = 24;
  auto ask_ahead = [&](int t) {
    if (kAhead == 1 || t >= end || ((t - begin) & 7) != warp) return;
    const int unit_lines = (8 * dim + 127) / 128;
    const char* where = nullptr;
    if (lane < unit_lines)
      where = reinterpret_cast<const char*>(scales + ((size_t)t * kv_heads + kv_head) * 2 * (size_t)dim) + lane * 128;
    else if (lane == unit_lines)
      where = reinterpret_cast<const char*>(qkv + (size_t)t * row_width + v_at);
    else if (lane == unit_lines + 1)
      where = reinterpret_cast<const char*>(gates + ((size_t)t * heads + head) * 2);
    if (where != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(where));
  };
  for (int t = begin; t < begin + kFar; ++t) ask_ahead(t);
#pragma unroll
  for (int a = 0; a < kAhead; ++a)
    if (begin + a < end) fetch(ring[a], begin + a);
  for (int t = begin; t < end; t += kAhead) {
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
      if (t + a < end) {
        ask_ahead(t + a + kFar);
        step(ring[a], t + a);
        if (t + a + kAhead < end) fetch(ring[a], t + a + kAhead);
      }
    }
  }
  {
    const float o = sum_over_column_lanes(o_parts) * o_scale;       // the last token's read-out
    if (live && part == 0) out[(size_t)o_token * heads * vdim + (size_t)head * vdim + column] = o;
  }

  if (!live) return;
  if (kVector) {
#pragma unroll
    for (int c = 0; c < R / 4; ++c)
      *reinterpret_cast<float4*>(mine + c * 4) = make_float4(S[c * 4], S[c * 4 + 1], S[c * 4 + 2], S[c * 4 + 3]);
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (r < mine_dims) mine[r] = S[r];
  }
}

// The same recurrence for prompts and portions, with the tokens' inputs staged in shared memory: the loads of a
// register ring several tokens deep share a warp's few scoreboards, so a wait for one token's inputs also waits
// for the ones just asked for, and a token cost a whole trip to the second-level cache (0.5 us, whatever the head
// size).  Here a block copies eight tokens at a time (unit q and k in float, gates, the block's 16 values of v)
// with cp.async, whose groups are waited for in order, two chunks in flight, and reads them with shared-memory
// loads.  For dim == 8 R, vdim a multiple of 16 and 16-byte aligned rows.
constexpr int kStageTokens = 8;

template <typename T, int R>
__global__ void __launch_bounds__(128)
gated_delta_rule_staged_kernel(const T* __restrict__ qkv, const float* __restrict__ units, const float* __restrict__ gates,
                               float* __restrict__ state, const int* __restrict__ query_start_loc,
                               const int* __restrict__ state_slots, float* __restrict__ out, int heads, int kv_heads,
                               int vdim) {
  // Four warps and 16 columns a block: a prompt alone is a few hundred chains (heads x vdim columns / 4 a warp),
  // fewer than the device has schedulers, so each warp gets a scheduler of its own and as little of a column's
  // arithmetic as the lanes of a column can share.
  extern __shared__ __align__(16) unsigned char staged[];
  constexpr int dim = 8 * R, kColumns = 16;
  constexpr int kUnitBytes = 8 * dim, kValueBytes = kColumns * (int)sizeof(T);
  constexpr int kTokenBytes = kUnitBytes + 16 + (kValueBytes + 15) / 16 * 16;   // units | gates (8 bytes, padded) | v
  constexpr int kCopies = kUnitBytes / 16 + 1 + kValueBytes / 16;               // per token: 16-byte copies, one of 8 for the gates
  grid_dependency_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int begin = query_start_loc[seq], end = query_start_loc[seq + 1];
  if (end <= begin) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane >> 2;
  const int local_column = warp * 4 + (lane & 3), column = blockIdx.x * kColumns + local_column;
  const int first = part * R;
  const int qk_width = kv_heads * dim;
  const size_t row_width = 2 * (size_t)qk_width + (size_t)heads * vdim;
  const int kv_head = head / (heads / kv_heads);
  const size_t v_at = 2 * (size_t)qk_width + (size_t)head * vdim + (size_t)blockIdx.x * kColumns;
  float* mine = state + (((size_t)state_slots[seq] * heads + head) * vdim + column) * dim + first;

  float S[R];
#pragma unroll
  for (int c = 0; c < R / 4; ++c) {
    const float4 v = *reinterpret_cast<const float4*>(mine + c * 4);
    S[c * 4] = v.x; S[c * 4 + 1] = v.y; S[c * 4 + 2] = v.z; S[c * 4 + 3] = v.w;
  }

  auto copy_chunk = [&](int chunk) {
    unsigned char* buffer = staged + (size_t)(chunk & 1) * kStageTokens * kTokenBytes;
    const int t0 = begin + chunk * kStageTokens;
    for (int i = threadIdx.x; i < kStageTokens * kCopies; i += 128) {
      const int j = i / kCopies, c = i - j * kCopies, t = t0 + j;
      if (t >= end) continue;
      unsigned char* dst = buffer + (size_t)j * kTokenBytes;
      if (c < kUnitBytes / 16) {
        const char* src = reinterpret_cast<const char*>(units + ((size_t)t * kv_heads + kv_head) * 2 * dim) + c * 16;
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst + c * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
      } else if (c == kUnitBytes / 16) {
        const char* src = reinterpret_cast<const char*>(gates + ((size_t)t * heads + head) * 2);
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst + kUnitBytes);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src));
      } else {
        const int k = c - kUnitBytes / 16 - 1;
        const char* src = reinterpret_cast<const char*>(qkv + (size_t)t * row_width + v_at) + k * 16;
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst + kUnitBytes + 16 + k * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
      }
    }
    asm volatile("cp.async.commit_group;" ::);
  };

  float o_parts = 0.f;
  int o_token = -1;
  const int chunks = (end - begin + kStageTokens - 1) / kStageTokens;
  copy_chunk(0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    if (chunk + 1 < chunks) {
      copy_chunk(chunk + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const unsigned char* buffer = staged + (size_t)(chunk & 1) * kStageTokens * kTokenBytes;
    const int t0 = begin + chunk * kStageTokens, count = min(kStageTokens, end - t0);
#pragma unroll 2
    for (int j = 0; j < count; ++j) {
      const unsigned char* tok = buffer + (size_t)j * kTokenBytes;
      const float* q = reinterpret_cast<const float*>(tok) + first;
      const float* k = q + dim;
      const float2 ga = *reinterpret_cast<const float2*>(tok + kUnitBytes);
      const float v = widen(reinterpret_cast<const T*>(tok + kUnitBytes + 16)[local_column]);
      float kk[R];
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k + r);
        kk[r] = k4.x; kk[r + 1] = k4.y; kk[r + 2] = k4.z; kk[r + 3] = k4.w;
        d0 = fmaf(S[r], k4.x, d0); d1 = fmaf(S[r + 1], k4.y, d1);
        d2 = fmaf(S[r + 2], k4.z, d2); d3 = fmaf(S[r + 3], k4.w, d3);
      }
      // The read-out of the token before is added up over the lanes together with this token's S^T k.
      float dsum = (d0 + d1) + (d2 + d3), osum = o_parts;
#pragma unroll
      for (int offset = 4; offset <= 16; offset <<= 1) {
        const float a = __shfl_xor_sync(0xffffffffu, dsum, offset), b = __shfl_xor_sync(0xffffffffu, osum, offset);
        dsum += a;
        osum += b;
      }
      if (o_token >= 0 && part == 0) out[(size_t)o_token * heads * vdim + (size_t)head * vdim + column] = osum;
      const float c = ga.x * (v - dsum * ga.y);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(q + r);
        S[r] = fmaf(S[r], ga.y, kk[r] * c); S[r + 1] = fmaf(S[r + 1], ga.y, kk[r + 1] * c);
        S[r + 2] = fmaf(S[r + 2], ga.y, kk[r + 2] * c); S[r + 3] = fmaf(S[r + 3], ga.y, kk[r + 3] * c);
        o0 = fmaf(S[r], q4.x, o0); o1 = fmaf(S[r + 1], q4.y, o1);
        o2 = fmaf(S[r + 2], q4.z, o2); o3 = fmaf(S[r + 3], q4.w, o3);
      }
      o_parts = (o0 + o1) + (o2 + o3);
      o_token = t0 + j;
    }
    __syncthreads();     // the buffer is written again two chunks on
  }
  {
    const float o = sum_over_column_lanes(o_parts);
    if (part == 0) out[(size_t)o_token * heads * vdim + (size_t)head * vdim + column] = o;
  }
#pragma unroll
  for (int c = 0; c < R / 4; ++c)
    *reinterpret_cast<float4*>(mine + c * 4) = make_float4(S[c * 4], S[c * 4 + 1], S[c * 4 + 2], S[c * 4 + 3]);
}

template <typename T, int R>
int launch_delta_r(bool single, bool vector, int tokens, dim3 grid, cudaStream_t stream, const T* qkv, const float* scales,
                   const float* gates, float* state, const int* qsl, const int* slots, float* out, int heads,
                   int kv_heads, int dim, int vdim, const T* ab, size_t ab_stride, const float* a_log,
                   const float* dt_bias) {
  // Tokens in flight: as many as the registers hold beside the state (a token costs 2 R + 5 of them).
  constexpr int kDeep = (2 * R + 5) * 4 + R <= 190 ? 4 : 2;
#define LI_DELTA(AHEAD, VEC)                                                                                          \
  return (int)launch_pdl(tokens, gated_delta_rule_kernel<T, R, AHEAD, VEC>, grid, dim3(256), 0, stream, qkv, scales,  \
                         gates, state, qsl, slots, out, heads, kv_heads, dim, vdim, ab, ab_stride, a_log, dt_bias)
  if (single) {
    if (vector) LI_DELTA(1, true);
    LI_DELTA(1, false);
  }
  if (vector && vdim % 16 == 0 && aligned16(scales) && (((size_t)heads * vdim) * sizeof(T)) % 16 == 0) {
    constexpr size_t smem = 2 * (size_t)kStageTokens * (8 * 8 * R + 16 + (16 * sizeof(T) + 15) / 16 * 16);
    const dim3 staged_grid(vdim / 16, grid.y, grid.z);
    return (int)launch_pdl(tokens, gated_delta_rule_staged_kernel<T, R>, staged_grid, dim3(128), smem, stream, qkv, scales, gates,
                           state, qsl, slots, out, heads, kv_heads, vdim);
  }
  if (vector) LI_DELTA(kDeep, true);
  LI_DELTA(kDeep, false);
#undef LI_DELTA
}

template <typename T>
int launch_delta(int dim, bool single, int tokens, dim3 grid, cudaStream_t stream, const T* qkv, const float* scales,
                 const float* gates, float* state, const int* qsl, const int* slots, float* out, int heads,
                 int kv_heads, int vdim, const T* ab, size_t ab_stride, const float* a_log, const float* dt_bias) {
  const int R = dim <= 32 ? 4 : dim <= 64 ? 8 : dim <= 128 ? 16 : 32;
  const size_t row_bytes = (2 * (size_t)kv_heads * dim + (size_t)heads * vdim) * sizeof(T);
  const bool vector = dim == 8 * R && row_bytes % 16 == 0 && aligned16(qkv) && aligned16(state) &&
                      (R * sizeof(T)) % 16 == 0;
#define LI_DELTA_R(RR)                                                                                                \
  return launch_delta_r<T, RR>(single, vector, tokens, grid, stream, qkv, scales, gates, state, qsl, slots, out, heads, \
                               kv_heads, dim, vdim, ab, ab_stride, a_log, dt_bias)
  if (R == 4) LI_DELTA_R(4);
  if (R == 8) LI_DELTA_R(8);
  if (R == 16) LI_DELTA_R(16);
  LI_DELTA_R(32);
#undef LI_DELTA_R
}

}  // namespace li

using namespace li;

LI_EXPORT int li_short_conv(int dtype, const void* x, size_t x_stride, const void* taps, const void* tail,
                            const int* seq_of_token, const int* query_start_loc, const int* state_slots, void* out,
                            int tokens, int channels, int K, int act, int move_tail, cudaStream_t stream) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (K < 1 || K > kMaxTaps || (K > 1 && tail == nullptr) || (channels + 127) / 128 > 65535) return LI_ERR_UNSUPPORTED;
  // move_tail: every sequence of the step brings exactly one token and the caller wants the tail moved on by
  // this launch; only the vector kernel does that (LI_ERR_UNSUPPORTED otherwise: the caller then updates apart).
  const int lanes = dtype == kFloat32 ? 4 : 8;     // channels in a 16-byte vector
  if (channels % lanes == 0 && x_stride % lanes == 0 && aligned16(x) && aligned16(out) && aligned16(taps) &&
      (K == 1 || aligned16(tail))) {
    const int vectors = channels / lanes;
    const dim3 vgrid(tokens, (vectors + 127) / 128);
    if (dtype == kFloat32)
      return (int)launch_pdl(tokens, short_conv_vec_kernel<float>, vgrid, dim3(128), 0, stream, (const float*)x, x_stride,
                             (const float*)taps, (const float*)tail, seq_of_token, query_start_loc, state_slots,
                             (float*)out, channels, K, act, move_tail ? (float*)tail : (float*)nullptr);
    return (int)launch_pdl(tokens, short_conv_vec_kernel<bf16>, vgrid, dim3(128), 0, stream, (const bf16*)x, x_stride,
                           (const bf16*)taps, (const bf16*)tail, seq_of_token, query_start_loc, state_slots, (bf16*)out,
                           channels, K, act, move_tail ? (bf16*)tail : (bf16*)nullptr);
  }
  if (move_tail) return LI_ERR_UNSUPPORTED;
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
// [slots, heads, vdim, dim] (column by column); out [tokens, heads * vdim]; scratch: 2 * tokens * (kv_heads * dim +
// heads) floats.  max_q_len: the most tokens a sequence brings (1 chooses the variant without tokens in flight).
LI_EXPORT int li_gated_delta_rule(int dtype, const void* qkv, const void* ab, size_t ab_stride, int tokens, int num_seqs,
                                  const float* a_log, const float* dt_bias, float* state, const int* query_start_loc,
                                  const int* state_slots, float* out, int heads, int kv_heads, int dim, int vdim,
                                  int max_q_len, float* scratch, cudaStream_t stream) {
  if (tokens <= 0 || num_seqs <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || dim > 256 || vdim < 1 || heads > 65535 ||
      num_seqs > 65535 || scratch == nullptr)
    return LI_ERR_UNSUPPORTED;
  float* scales = scratch;
  float* gates = scratch + 2 * (size_t)tokens * kv_heads * dim;
  const size_t row_width = 2 * (size_t)kv_heads * dim + (size_t)heads * vdim;
  const size_t items = (size_t)tokens * (kv_heads + (heads + 31) / 32);
  const dim3 gates_grid((unsigned)((items + 7) / 8));
  const dim3 grid((vdim + 31) / 32, heads, num_seqs);
  const bool single = max_q_len == 1;     // the recurrence kernel then works out scales and gates itself
  int code = 0;
  if (dtype == kFloat32) {
    if (!single)
      code = (int)launch_pdl(tokens, delta_gates_kernel<float>, gates_grid, dim3(256), 0, stream, (const float*)qkv,
                             row_width, (const float*)ab, ab_stride, a_log, dt_bias, scales, gates, tokens, heads,
                             kv_heads, dim);
    if (code) return code;
    return launch_delta<float>(dim, single, tokens, grid, stream, (const float*)qkv, scales, gates, state,
                               query_start_loc, state_slots, out, heads, kv_heads, vdim, (const float*)ab, ab_stride,
                               a_log, dt_bias);
  }
  if (!single)
    code = (int)launch_pdl(tokens, delta_gates_kernel<bf16>, gates_grid, dim3(256), 0, stream, (const bf16*)qkv,
                           row_width, (const bf16*)ab, ab_stride, a_log, dt_bias, scales, gates, tokens, heads, kv_heads,
                           dim);
  if (code) return code;
  return launch_delta<bf16>(dim, single, tokens, grid, stream, (const bf16*)qkv, scales, gates, state, query_start_loc,
                            state_slots, out, heads, kv_heads, vdim, (const bf16*)ab, ab_stride, a_log, dt_bias);
}
