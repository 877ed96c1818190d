// A residual kept as several 32-bit streams ("hyper-connections"), and the root-mean-square norm that reads it.
//
// The residual of a token is S copies x_1..x_S of `width` floats, side by side in one row [S * width] (S = 1 is
// the ordinary single residual).  A sublayer reads u = sum_s read[s] x_s, is fed norm(u), and its output y
// rewrites all streams at once from the old ones:
//
//     x_t <- sum_s mix[s, t] x_s + write[t] * gain * y          (gain: one factor per channel, "layer scale")
//
// One kernel does what lies between two sublayers: the rewrite that the sublayer before left pending, the read
// of the sublayer after it, and that sublayer's norm  out = u / sqrt(mean(u^2) + eps) * weight * out_scale,
// so the streams are read and written once per sublayer.  Everything is 32-bit; only y (the sublayer's output)
// and out (the next sublayer's input) have the engine's dtype.  With `rows` only those rows are produced and the
// rewrite is not stored (the model's last norm, which reads the sum of the streams: read = null).
//
// The embedding that starts the streams: every copy = table[id] * scale, widened before the multiply.
#include "common.cuh"

namespace li {

constexpr int kMaxStreams = 8;

template <typename T>
__global__ void embedding_streams_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                         float* __restrict__ out, int width, int vocab, float scale, int copies,
                                         int* __restrict__ error_flag) {
  const int t = blockIdx.x;
  grid_dependency_wait();
  grid_launch_dependents();
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) *error_flag = 1;
  const T* row = table + (size_t)(ok ? id : 0) * width;
  float* o = out + (size_t)t * copies * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = ok ? __fmul_rn(to_float(row[d]), scale) : 0.f;
    for (int s = 0; s < copies; ++s) o[(size_t)s * width + d] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
stream_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain,
                      const float* __restrict__ write, const float* __restrict__ mix,
                      const float* __restrict__ read, const float* __restrict__ weight, T* __restrict__ out,
                      const int* __restrict__ rows, int width, int S, float eps, float out_scale, int store) {
  extern __shared__ __align__(16) float u_smem[];     // [width] the read-out of this row, then scratch for the block's sum
  __shared__ float coeff[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  __shared__ float scratch[33];
  float* mix_s = coeff;
  float* write_s = coeff + kMaxStreams * kMaxStreams;
  float* read_s = write_s + kMaxStreams;
  // The coefficients are weights: they may be fetched before the kernel ahead has finished.
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = (y != nullptr) ? mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    write_s[i] = (y != nullptr) ? write[i] : 0.f;
    read_s[i] = read ? read[i] : 1.0f;
  }
  grid_dependency_wait();
  grid_launch_dependents();
  __syncthreads();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * S * width;
  const T* yr = y ? y + (size_t)row * width : nullptr;
  float sumsq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float old[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) old[s] = s < S ? xr[(size_t)s * width + d] : 0.f;
    float u = 0.f;
    if (yr) {
      const float add = __fmul_rn(gain ? gain[d] : 1.0f, to_float(yr[d]));
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t >= S) break;
        float v = __fmul_rn(write_s[t], add);
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) v = fmaf(mix_s[s * S + t], old[s], v);
        if (store) xr[(size_t)t * width + d] = v;
        u = fmaf(read_s[t], v, u);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) u = fmaf(read_s[s], old[s], u);
    }
    u_smem[d] = u;
    sumsq = fmaf(u, u, sumsq);
  }
  if (!out) return;
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)width + eps);
  T* o = out + (size_t)r * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    o[d] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(u_smem[d], inv), weight[d]), out_scale));
}

// The same for a known number of streams and a width that is a multiple of four: every thread takes four
// neighbouring channels at a time (16-byte accesses to every stream), the small sums are unrolled.
template <typename T, int S>
__global__ void __launch_bounds__(256)
stream_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gain,
                          const float* __restrict__ write, const float* __restrict__ mix,
                          const float* __restrict__ read, const float* __restrict__ weight, T* __restrict__ out,
                          const int* __restrict__ rows, int width, float eps, float out_scale, int store) {
  extern __shared__ __align__(16) float u_smem[];
  __shared__ float scratch[33];
  float mix_r[S][S], write_r[S], read_r[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    write_r[s] = y ? write[s] : 0.f;
    read_r[s] = read ? read[s] : 1.0f;
#pragma unroll
    for (int t = 0; t < S; ++t) mix_r[s][t] = y ? mix[s * S + t] : 0.f;
  }
  grid_dependency_wait();
  grid_launch_dependents();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * S * width;
  const T* yr = y ? y + (size_t)row * width : nullptr;
  float sumsq = 0.f;
  for (int d = threadIdx.x * 4; d < width; d += blockDim.x * 4) {
    float4 old[S];
#pragma unroll
    for (int s = 0; s < S; ++s) old[s] = *reinterpret_cast<const float4*>(xr + (size_t)s * width + d);
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    if (yr) {
      float add[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) add[e] = __fmul_rn(gain ? gain[d + e] : 1.0f, to_float(yr[d + e]));
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[e] = __fmul_rn(write_r[t], add[e]);
#pragma unroll
          for (int s = 0; s < S; ++s) v[e] = fmaf(mix_r[s][t], (&old[s].x)[e], v[e]);
          u[e] = fmaf(read_r[t], v[e], u[e]);
        }
        if (store) *reinterpret_cast<float4*>(xr + (size_t)t * width + d) = make_float4(v[0], v[1], v[2], v[3]);
      }
    } else {
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int e = 0; e < 4; ++e) u[e] = fmaf(read_r[s], (&old[s].x)[e], u[e]);
    }
    *reinterpret_cast<float4*>(u_smem + d) = make_float4(u[0], u[1], u[2], u[3]);
#pragma unroll
    for (int e = 0; e < 4; ++e) sumsq = fmaf(u[e], u[e], sumsq);
  }
  if (!out) return;
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)width + eps);
  T* o = out + (size_t)r * width;
  for (int d = threadIdx.x * 4; d < width; d += blockDim.x * 4) {
    const float4 u = *reinterpret_cast<const float4*>(u_smem + d);
    const float4 w = *reinterpret_cast<const float4*>(weight + d);
    o[d] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(u.x, inv), w.x), out_scale));
    o[d + 1] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(u.y, inv), w.y), out_scale));
    o[d + 2] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(u.z, inv), w.z), out_scale));
    o[d + 3] = from_float<T>(__fmul_rn(__fmul_rn(__fmul_rn(u.w, inv), w.w), out_scale));
  }
}

template <typename T, int S>
cudaError_t launch_stream_vec(int n, size_t smem, cudaStream_t stream, float* x, const void* y, const float* gain,
                              const float* write, const float* mix, const float* read, const float* weight, void* out,
                              const int* rows, int width, float eps, float out_scale, int store) {
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(stream_rmsnorm_vec_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int threads = width >= 1024 ? 256 : 128;
  return launch_pdl(n, stream_rmsnorm_vec_kernel<T, S>, dim3(n), dim3(threads), smem, stream, x, (const T*)y, gain,
                    write, mix, read, weight, (T*)out, rows, width, eps, out_scale, store);
}

template <typename T>
cudaError_t launch_stream_vec_any(int S, int n, size_t smem, cudaStream_t stream, float* x, const void* y,
                                  const float* gain, const float* write, const float* mix, const float* read,
                                  const float* weight, void* out, const int* rows, int width, float eps,
                                  float out_scale, int store) {
#define LI_STREAMS(N) case N: return launch_stream_vec<T, N>(n, smem, stream, x, y, gain, write, mix, read, weight, out, rows, width, eps, out_scale, store);
  switch (S) {
    LI_STREAMS(1) LI_STREAMS(2) LI_STREAMS(3) LI_STREAMS(4) LI_STREAMS(5) LI_STREAMS(6) LI_STREAMS(7) LI_STREAMS(8)
  }
#undef LI_STREAMS
  return cudaErrorInvalidValue;
}

}  // namespace li

using namespace li;

// out[t, s, :] = float(table[ids[t]]) * scale for every copy s; an id outside the table gives zeros and raises the flag.
LI_EXPORT int li_embedding_streams(int dtype, const int* ids, const void* table, float* out, int tokens, int width,
                                   int vocab, float scale, int copies, int* error_flag, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (copies < 1 || copies > kMaxStreams) return LI_ERR_UNSUPPORTED;
  const int threads = width >= 256 ? 256 : 128;
  cudaError_t e;
  if (dtype == kFloat32)
    e = launch_pdl(tokens, embedding_streams_kernel<float>, dim3(tokens), dim3(threads), 0, stream, ids,
                   (const float*)table, out, width, vocab, scale, copies, error_flag);
  else
    e = launch_pdl(tokens, embedding_streams_kernel<bf16>, dim3(tokens), dim3(threads), 0, stream, ids,
                   (const bf16*)table, out, width, vocab, scale, copies, error_flag);
  return (int)e;
}

// x [tokens, S * width] float (read; written when y and store); y [tokens, width] or null (no rewrite pending);
// gain [width] or null; write [S], mix [S, S] ([from, to]); read [S] or null (all ones); weight [width] float;
// out [n, width] in the engine's dtype (null: only the rewrite); rows [n] or null (row r of out is row r of x).
LI_EXPORT int li_stream_rmsnorm(int dtype, float* x, const void* y, const float* gain, const float* write,
                                const float* mix, const float* read, const float* weight, void* out, const int* rows,
                                int n, int width, int S, float eps, float out_scale, int store, cudaStream_t stream) {
  if (n == 0) return 0;
  if (S < 1 || S > kMaxStreams || width < 1) return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return LI_ERR_UNSUPPORTED;
  cudaError_t e;
  if (width % 4 == 0 && aligned16(x) && (!weight || aligned16(weight))) {
    e = dtype == kFloat32
            ? launch_stream_vec_any<float>(S, n, smem, stream, x, y, gain, write, mix, read, weight, out, rows, width, eps, out_scale, store)
            : launch_stream_vec_any<bf16>(S, n, smem, stream, x, y, gain, write, mix, read, weight, out, rows, width, eps, out_scale, store);
    return (int)e;
  }
  if (dtype == kFloat32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(n, stream_rmsnorm_kernel<float>, dim3(n), dim3(256), smem, stream, x, (const float*)y, gain, write,
                   mix, read, weight, (float*)out, rows, width, S, eps, out_scale, store);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = launch_pdl(n, stream_rmsnorm_kernel<bf16>, dim3(n), dim3(256), smem, stream, x, (const bf16*)y, gain, write,
                   mix, read, weight, (bf16*)out, rows, width, S, eps, out_scale, store);
  }
  return (int)e;
}
