// Row kernels of models whose residual stream is float32 on every path: a scaled
// embedding gather, RMSNorm over a float32 stream with the residual add folded in,
// and the gated activation of a feed-forward with the activation as an argument.
//
// Norm: s = x + m * (branch + branch2) (float32, written out as the new stream; the second
// branch is optional and m is 1 for the usual add); y = s * rsqrt(mean(s^2) + eps) *
// (offset + w), rounded once to the element type T of the path; a second gain gives a
// second result from the same pass. The gains are float32. One block per row, the row
// held in shared memory, global memory read once.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embed_scaled_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                    int H, int n_table_rows, float scale, int* error, int copies) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int id = ids[r];
  const bool bad = id < 0 || id >= n_table_rows;
  if (bad && threadIdx.x == 0 && error) atomicExch(error, 1);
  const T* src = table + (size_t)(bad ? 0 : id) * H;
  float* dst = out + (size_t)r * H * copies;  // the row is written `copies` times side by side
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = bad ? 0.f : to_float<T>(src[i]) * scale;
    for (int c = 0; c < copies; ++c) dst[(size_t)c * H + i] = v;
  }
}

template <typename T> __device__ __forceinline__ void load4_rows(const T* p, float* f);
template <> __device__ __forceinline__ void load4_rows<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4_rows<bf16>(const bf16* p, float* f) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  f[0] = __low2float(h[0]); f[1] = __high2float(h[0]); f[2] = __low2float(h[1]); f[3] = __high2float(h[1]);
}
template <typename T> __device__ __forceinline__ void store4_rows(T* p, const float* f);
template <> __device__ __forceinline__ void store4_rows<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4_rows<bf16>(bf16* p, const float* f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, bool VEC>
__global__ void rmsnorm_wide_kernel(T* __restrict__ out, float* x_new, const float* x, const T* __restrict__ branch,
                                    const float* __restrict__ gain, float offset, int H, float eps,
                                    const T* __restrict__ branch2, float bscale, const float* __restrict__ gain2,
                                    T* __restrict__ out2) {
  extern __shared__ __align__(16) float row_s[];  // H floats
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t base = (size_t)blockIdx.x * H;
  float sq = 0.f;
  if (VEC) {  // H a multiple of 4: 16-byte pieces of the stream, 8- or 16-byte pieces of the branch and the result
    const float4* xv = reinterpret_cast<const float4*>(x + base);
    float4* nv = reinterpret_cast<float4*>(x_new + base);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      float4 f = xv[i];
      if (branch) {
        float b[4];
        load4_rows<T>(branch + base + 4 * i, b);
        if (branch2) {
          float c[4];
          load4_rows<T>(branch2 + base + 4 * i, c);
          b[0] += c[0]; b[1] += c[1]; b[2] += c[2]; b[3] += c[3];
        }
        f.x += bscale * b[0]; f.y += bscale * b[1]; f.z += bscale * b[2]; f.w += bscale * b[3];
        nv[i] = f;
      }
      reinterpret_cast<float4*>(row_s)[i] = f;
      sq += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float f = x[base + i];
      if (branch) {
        float b = to_float<T>(branch[base + i]);
        if (branch2) b += to_float<T>(branch2[base + i]);
        f += bscale * b;
        x_new[base + i] = f;
      }
      row_s[i] = f;
      sq += f * f;
    }
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
  if (VEC) {
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) {
      const float4 f = reinterpret_cast<const float4*>(row_s)[i];
      const float4 g = reinterpret_cast<const float4*>(gain)[i];
      const float r[4] = {f.x * rstd * (offset + g.x), f.y * rstd * (offset + g.y), f.z * rstd * (offset + g.z),
                          f.w * rstd * (offset + g.w)};
      store4_rows<T>(out + base + 4 * i, r);
      if (gain2) {
        const float4 h = reinterpret_cast<const float4*>(gain2)[i];
        const float r2[4] = {f.x * rstd * (offset + h.x), f.y * rstd * (offset + h.y), f.z * rstd * (offset + h.z),
                             f.w * rstd * (offset + h.w)};
        store4_rows<T>(out2 + base + 4 * i, r2);
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      out[base + i] = from_float<T>(row_s[i] * rstd * (offset + gain[i]));
      if (gain2) out2[base + i] = from_float<T>(row_s[i] * rstd * (offset + gain2[i]));
    }
  }
}

__device__ __forceinline__ float activation(float z, int act) {
  if (act == 0) return z / (1.0f + expf(-z));                                                   // silu
  if (act == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));  // gelu, tanh form
  return 1.0f / (1.0f + expf(-z));                                                              // sigmoid
}

// act 3: both inputs are clamped first, g' = min(g, limit), u' = clamp(u, -limit, limit), and the result is
// g' * sigmoid(slope * g') * (u' + 1)
__device__ __forceinline__ float gated(float g, float u, int act, float limit, float slope) {
  if (act != 3) return activation(g, act) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
}

// out[r, i] = round(act(g) * u), g = gu[r, i], u = gu[r, I + i]; with row_gate_col >= 0 the row is also
// multiplied by sigmoid(gu[r, row_gate_col]) (a gate of one number per row that rides in the same product)
template <typename T, bool VEC>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ gu, int gu_stride, int I, int act,
                                 int row_gate_col, float limit, float slope) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t r = blockIdx.x;
  const float rg = row_gate_col >= 0 ? activation(to_float<T>(gu[r * gu_stride + row_gate_col]), 2) : 1.f;
  if (VEC) {  // I and the row stride multiples of 4
    for (int i = 4 * (blockIdx.y * blockDim.x + threadIdx.x); i < I; i += 4 * gridDim.y * blockDim.x) {
      float g[4], u[4], o[4];
      load4_rows<T>(gu + r * gu_stride + i, g);
      load4_rows<T>(gu + r * gu_stride + I + i, u);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = gated(g[j], u[j], act, limit, slope) * rg;
      store4_rows<T>(out + r * I + i, o);
    }
    return;
  }
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < I; i += gridDim.y * blockDim.x) {
    const float g = to_float<T>(gu[r * gu_stride + i]);
    const float u = to_float<T>(gu[r * gu_stride + I + i]);
    out[r * I + i] = from_float<T>(gated(g, u, act, limit, slope) * rg);
  }
}

}  // namespace

KRK_API int krk_embed_scaled(float* out, const void* table, const int* ids, int rows, int H, int n_table_rows, float scale,
                             int* error, int dtype, cudaStream_t stream, int copies) {
  if (rows == 0) return 0;
  if (copies < 1) return -2;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(embed_scaled_kernel<float>, dim3(rows), dim3(128), 0, stream, out, (const float*)table, ids, H,
                           n_table_rows, scale, error, copies);
  return (int)launch_pdl(embed_scaled_kernel<bf16>, dim3(rows), dim3(128), 0, stream, out, (const bf16*)table, ids, H,
                         n_table_rows, scale, error, copies);
}

template <typename T>
static int launch_rmsnorm_wide(void* out, float* x_new, const float* x, const void* branch, const float* gain,
                               float offset, int rows, int H, float eps, const void* branch2, float bscale,
                               const float* gain2, void* out2, cudaStream_t stream) {
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 220 * 1024) return -2;
  const int threads = H >= 4096 ? 1024 : (H >= 1024 ? 256 : 128);
  const bool vec = H % 4 == 0 && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)gain2 & 15) == 0;
  auto kern = vec ? rmsnorm_wide_kernel<T, true> : rmsnorm_wide_kernel<T, false>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (T*)out, x_new, x, (const T*)branch, gain, offset,
                         H, eps, (const T*)branch2, bscale, gain2, (T*)out2);
}

KRK_API int krk_rmsnorm_wide(void* out, float* x_new, const float* x, const void* branch, const float* gain, float offset,
                             int rows, int H, float eps, const void* branch2, float bscale, const float* gain2, void* out2,
                             int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (!branch && branch2) return -2;
  return dtype == KRK_DTYPE_F32
             ? launch_rmsnorm_wide<float>(out, x_new, x, branch, gain, offset, rows, H, eps, branch2, bscale, gain2, out2, stream)
             : launch_rmsnorm_wide<bf16>(out, x_new, x, branch, gain, offset, rows, H, eps, branch2, bscale, gain2, out2, stream);
}

KRK_API int krk_gated_act(void* out, const void* gu, int gu_stride, int rows, int I, int act, int row_gate_col, int dtype,
                          cudaStream_t stream, float limit, float slope) {
  if (rows == 0) return 0;
  const size_t esz = dtype == KRK_DTYPE_F32 ? 4 : 2;
  const bool vec = I % 4 == 0 && gu_stride % 4 == 0 && ((uintptr_t)gu & (4 * esz - 1)) == 0;
  const int chunks = min(64, (I / (vec ? 4 : 1) + 255) / 256);
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(vec ? gated_act_kernel<float, true> : gated_act_kernel<float, false>, dim3(rows, chunks),
                           dim3(256), 0, stream, (float*)out, (const float*)gu, gu_stride, I, act, row_gate_col, limit, slope);
  return (int)launch_pdl(vec ? gated_act_kernel<bf16, true> : gated_act_kernel<bf16, false>, dim3(rows, chunks), dim3(256),
                         0, stream, (bf16*)out, (const bf16*)gu, gu_stride, I, act, row_gate_col, limit, slope);
}
