// Row kernels of models with several residual streams (hyper-connections), and the biases and whole-row norms
// of an attention's projections.
//
// krk_hyper_rmsnorm: a token's S streams lie side by side in one float32 row [S * C]. With a pending output y
// [C] of the sublayer before and that sublayer's M [S, S] (indexed [from, to]) and b [S], the streams are
// rewritten, all from the old ones, x_t <- sum_s M[s, t] x_s + b_t y, and stored. Then u = sum_s a_s x_s with
// the next sublayer's a [S], and out = u * rsqrt(mean(u^2) + eps) * (offset + gain), rounded once to the
// path's type. Everything else is float32. One block per row; u is held in shared memory.
//
// krk_bias_row_norm: in place on the rows of a stacked q | k | v product: the biases are added, the q columns
// (all heads together) are divided by their root mean square and multiplied by a weight of their size, the k
// columns likewise, in float32, and the row is rounded back to the path's type.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

template <typename T, int V> struct alignas(V * sizeof(T)) Run { T v[V]; };

// V: elements a thread takes at a time (4 where C is a multiple of 4: 16-byte pieces of the streams)
template <typename T, int V>
__global__ void hyper_rmsnorm_kernel(T* __restrict__ out, float* x_new, const float* x, const T* __restrict__ branch,
                                     const float* __restrict__ fold, const float* __restrict__ read,
                                     const float* __restrict__ gain, float offset, int S, int C, float eps) {
  extern __shared__ __align__(16) float u_s[];  // C floats
  __shared__ float scratch[32];
  __shared__ float w_s[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
  grid_launch_dependents();
  float* M = w_s;                  // [from][to]
  float* b = w_s + S * S;          // [to]
  float* a = w_s + S * S + S;      // [from]
  if (threadIdx.x < S * S + S) w_s[threadIdx.x] = branch ? fold[threadIdx.x] : 0.f;  // weights: no kernel writes them
  if (threadIdx.x < S) a[threadIdx.x] = read[threadIdx.x];
  __syncthreads();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * S * C;
  float sq = 0.f;
  for (int c = V * threadIdx.x; c < C; c += V * blockDim.x) {
    Run<float, V> xs[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s)
      if (s < S) xs[s] = *reinterpret_cast<const Run<float, V>*>(x + base + (size_t)s * C + c);
    Run<float, V> u;
#pragma unroll
    for (int k = 0; k < V; ++k) u.v[k] = 0.f;
    if (branch) {
      const Run<T, V> y = *reinterpret_cast<const Run<T, V>*>(branch + (size_t)blockIdx.x * C + c);
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) {
        if (t < S) {
          Run<float, V> v;
#pragma unroll
          for (int k = 0; k < V; ++k) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
              if (s < S) acc += M[s * S + t] * xs[s].v[k];
            acc += b[t] * to_float<T>(y.v[k]);
            v.v[k] = acc;
            u.v[k] += a[t] * acc;
          }
          *reinterpret_cast<Run<float, V>*>(x_new + base + (size_t)t * C + c) = v;
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) {
#pragma unroll
          for (int k = 0; k < V; ++k) u.v[k] += a[s] * xs[s].v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      u_s[c + k] = u.v[k];
      sq += u.v[k] * u.v[k];
    }
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)C + eps);
  for (int c = V * threadIdx.x; c < C; c += V * blockDim.x) {
    Run<T, V> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_float<T>(u_s[c + k] * rstd * (offset + gain[c + k]));
    *reinterpret_cast<Run<T, V>*>(out + (size_t)blockIdx.x * C + c) = o;
  }
}

// one block per row; columns q0 .. k0 are the q row, k0 .. v0 the k row, v0 .. end the v row. A thread takes V
// consecutive elements at a time (V = 1, or 16 bytes of the row where the three parts' sizes, the row stride and
// the addresses are multiples of that: a piece then lies in one part).
template <typename T, int V>
__global__ void bias_row_norm_kernel(T* proj, int stride, int q0, int k0, int v0, int end,
                                     const float* __restrict__ bias, const float* __restrict__ gain, float eps) {
  extern __shared__ __align__(16) float row_s[];  // end - q0 floats
  __shared__ float scratch[32];
  constexpr int W = V >= 4 ? 4 : 1;  // the float32 vectors' pieces
  grid_launch_dependents();
  grid_dependency_wait();
  T* row = proj + (size_t)blockIdx.x * stride + q0;
  const int nq = k0 - q0, nk = v0 - k0, n = end - q0;
  float sq_q = 0.f, sq_k = 0.f;
  for (int i = V * threadIdx.x; i < n; i += V * blockDim.x) {
    const Run<T, V> raw = *reinterpret_cast<const Run<T, V>*>(row + i);
    float v[V], sq = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k) v[k] = to_float<T>(raw.v[k]);
    if (bias) {
#pragma unroll
      for (int k = 0; k < V; k += W) {
        const Run<float, W> b = *reinterpret_cast<const Run<float, W>*>(bias + i + k);
#pragma unroll
        for (int m = 0; m < W; ++m) v[k + m] += b.v[m];
      }
    }
#pragma unroll
    for (int k = 0; k < V; k += W) {
      Run<float, W> o;
#pragma unroll
      for (int m = 0; m < W; ++m) {
        o.v[m] = v[k + m];
        sq += v[k + m] * v[k + m];
      }
      *reinterpret_cast<Run<float, W>*>(row_s + i + k) = o;
    }
    if (i < nq) sq_q += sq;
    else if (i < nq + nk) sq_k += sq;
  }
  float rq = 1.f, rk = 1.f;
  if (gain) {
    rq = rsqrtf(block_sum(sq_q, scratch) / (float)nq + eps);
    rk = rsqrtf(block_sum(sq_k, scratch) / (float)nk + eps);
  } else {
    __syncthreads();
  }
  for (int i = V * threadIdx.x; i < n; i += V * blockDim.x) {  // every thread reads back what it wrote
    Run<T, V> o;
    const bool normed = gain && i < nq + nk;
    const float r = i < nq ? rq : rk;
#pragma unroll
    for (int k = 0; k < V; k += W) {
      const Run<float, W> v = *reinterpret_cast<const Run<float, W>*>(row_s + i + k);
      Run<float, W> g;
#pragma unroll
      for (int m = 0; m < W; ++m) g.v[m] = 1.f;
      if (normed) g = *reinterpret_cast<const Run<float, W>*>(gain + i + k);
#pragma unroll
      for (int m = 0; m < W; ++m) o.v[k + m] = from_float<T>(normed ? v.v[m] * r * g.v[m] : v.v[m]);
    }
    *reinterpret_cast<Run<T, V>*>(row + i) = o;
  }
}

}  // namespace

KRK_API int krk_hyper_rmsnorm(void* out, float* x_new, const float* x, const void* branch, const float* fold,
                              const float* read, const float* gain, float offset, int rows, int S, int C, float eps,
                              int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (S < 1 || S > MAX_STREAMS || (branch && !fold)) return -2;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int threads = C >= 4096 ? 512 : (C >= 1024 ? 256 : 128);
  const bool vec = C % 4 == 0;  // rows of the streams, the pending output and the result then start on 16 (8) bytes
  if (dtype == KRK_DTYPE_F32) {
    auto kern = vec ? hyper_rmsnorm_kernel<float, 4> : hyper_rmsnorm_kernel<float, 1>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (float*)out, x_new, x, (const float*)branch, fold,
                           read, gain, offset, S, C, eps);
  }
  auto kern = vec ? hyper_rmsnorm_kernel<bf16, 4> : hyper_rmsnorm_kernel<bf16, 1>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (bf16*)out, x_new, x, (const bf16*)branch, fold,
                         read, gain, offset, S, C, eps);
}

KRK_API int krk_bias_row_norm(void* proj, int stride, int q0, int k0, int v0, int end, const float* bias,
                              const float* gain, float eps, int rows, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (!(q0 < k0 && k0 < v0 && v0 <= end)) return -2;
  const int n = end - q0;
  const size_t smem = (size_t)n * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int V = dtype == KRK_DTYPE_F32 ? 4 : 8;
  const bool vec = (k0 - q0) % V == 0 && (v0 - k0) % V == 0 && n % V == 0 && stride % V == 0 && q0 % V == 0 &&
                   (((uintptr_t)proj | (uintptr_t)bias | (uintptr_t)gain) & 15) == 0;
  const int pieces = vec ? n / V : n;
  const int threads = pieces >= 4096 ? 512 : (pieces >= 1024 ? 256 : 128);
  if (dtype == KRK_DTYPE_F32) {
    auto kern = vec ? bias_row_norm_kernel<float, 4> : bias_row_norm_kernel<float, 1>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (float*)proj, stride, q0, k0, v0, end, bias,
                           gain, eps);
  }
  auto kern = vec ? bias_row_norm_kernel<bf16, 8> : bias_row_norm_kernel<bf16, 1>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (bf16*)proj, stride, q0, k0, v0, end, bias, gain,
                         eps);
}
