// Kernels of a feed-forward of routed experts.
//
// krk_moe_route: one warp per row. z = logits[r, :] + bias (float32); the `top` largest are taken one after
// the other (ties: the lower index), and their weights are the softmax over the chosen logits alone, or
// (`over_all`) each chosen expert's share of the softmax over all experts, which do not sum to one. A gate of one
// number per row may ride in the router's product as its last column: sigmoid of it is written beside the routing and
// multiplies what the experts' sum is added onto (a shared expert's output). (The router's product inside this
// kernel, one block per row, was measured for single-token steps and lost to the product kernel before it: 1.72
// against 1.53 ms a step of one sequence at 64 experts of width 2,048.)
//
// krk_moe_route_groups: the same walk over other scores (sigmoid scores, a stored correction for the choice, groups of
// experts of which only the best may be chosen); see moe_route_groups_kernel.
//
// Few rows (single-token steps): a (row, chosen expert) pair reads its expert's weights once.
//   krk_moe_gate_up_pairs: act[pair, f] = a(Wg_e[f] . x_r) * (Wu_e[f] . x_r), a warp per f, lanes over K.
//   krk_moe_down_pairs: out[r, c] = add[r, c] + sum_j weight[r, j] * (Wd_e(j)[c] . act[(r, j)]), a warp per c;
//   the sum over the chosen experts is float32, in the order of the choice.
//
// Many rows: pairs are counted per expert and ordered by expert on the device (krk_moe_sort: one block; offsets
// and the pairs' places), krk_moe_gather copies the rows into that order, the experts' products run over
// contiguous rows, and krk_moe_combine adds each row's weighted results onto `add`. With cap > 0 every expert's
// rows start at a multiple of cap (expert e's i-th pair sits in row e * cap + i), which is the layout a batched
// product over [experts, cap, K] reads.
#include "common.cuh"

namespace {

__device__ __forceinline__ float act_of(float z, int act) {
  if (act == 0) return z / (1.0f + expf(-z));
  if (act == 1) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return 1.0f / (1.0f + expf(-z));
}

constexpr int ROUTE_WARPS = 4;

// One warp: the `top` largest of z[0..E) one after the other (z is the warp's own shared memory and is consumed),
// their softmax weights.
__device__ __forceinline__ void route_row(float* z, int E, int top, int lane, int* __restrict__ experts,
                                          float* __restrict__ weights, int over_all) {
  float first = 0.f, total = 0.f, mine = 0.f;
  int mine_e = 0;
  float all = 0.f;
  if (over_all) {  // the denominator over every expert, before the walk consumes z
    float big = -INFINITY;
    for (int e = lane; e < E; e += 32) big = fmaxf(big, z[e]);
    big = warp_max(big);
    for (int e = lane; e < E; e += 32) all += expf(z[e] - big);
    all = warp_sum(all);
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; best_e = e; }  // ascending e: the lower index stays on a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (j == 0) first = best;
    const float p = expf(best - first);
    total += p;
    if (lane == j) { mine = p; mine_e = best_e; }
    if (lane == 0) z[best_e] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    experts[lane] = mine_e;
    weights[lane] = mine / (over_all ? all : total);  // the largest logit is the first one taken
  }
}

// logits [rows, E + has_gate]: the last column, if there is one, is a gate's logit of the row (it rides in the router's
// product), and sigmoid of it goes to row_gate
__global__ void moe_route_kernel(int* __restrict__ experts, float* __restrict__ weights, float* __restrict__ row_gate,
                                 const float* __restrict__ logits, const float* __restrict__ bias, int rows, int E,
                                 int has_gate, int top, int over_all) {
  extern __shared__ float z_s[];  // [warps][E]
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROUTE_WARPS + warp;
  if (row >= rows) return;
  float* z = z_s + (size_t)warp * E;
  const float* src = logits + (size_t)row * (E + has_gate);
  for (int e = lane; e < E; e += 32) z[e] = src[e] + (bias ? bias[e] : 0.f);
  if (has_gate && lane == 0) row_gate[row] = act_of(src[E], 2);
  __syncwarp();
  route_row(z, E, top, lane, experts + (size_t)row * top, weights + (size_t)row * top, over_all);
}

// The largest of z[0..n) over a warp (ties: the lower index).
__device__ __forceinline__ void warp_argmax(const float* z, int n, int lane, float* best_out, int* best_e_out) {
  float best = -INFINITY;
  int best_e = 0x7fffffff;
  for (int e = lane; e < n; e += 32) {
    const float v = z[e];
    if (v > best) { best = v; best_e = e; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
    if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
  }
  *best_out = best;
  *best_e_out = best_e;
}

// Sigmoid scores chosen within the best groups: s = sigmoid(logit); the choice goes by c = s + correction; the experts
// are `groups` equal runs of neighbours, a group's score is the sum of its two largest c (its one c where a group has one
// expert), only the `keep` best groups' experts can be chosen; the weights are the chosen s / (their sum + 1e-20) * scale.
__global__ void moe_route_groups_kernel(int* __restrict__ experts, float* __restrict__ weights, float* __restrict__ row_gate,
                                        const float* __restrict__ logits, const float* __restrict__ correction, int rows,
                                        int E, int has_gate, int top, int groups, int keep, float scale) {
  extern __shared__ float z_s[];  // [warps][2 E + 2 groups]
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROUTE_WARPS + warp;
  if (row >= rows) return;
  float* c = z_s + (size_t)warp * (2 * E + 2 * groups);
  float* s = c + E;
  float* gs = s + E;
  int* kept = reinterpret_cast<int*>(gs + groups);
  const float* src = logits + (size_t)row * (E + has_gate);
  for (int e = lane; e < E; e += 32) {
    const float v = act_of(src[e], 2);
    s[e] = v;
    c[e] = v + correction[e];
  }
  if (has_gate && lane == 0) row_gate[row] = act_of(src[E], 2);
  __syncwarp();
  if (keep < groups) {
    const int size = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;  // the largest and the second largest
      for (int e = g * size; e < (g + 1) * size; ++e) {
        const float v = c[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = size > 1 ? a + b : a;
      kept[g] = 0;
    }
    __syncwarp();
    for (int j = 0; j < keep; ++j) {
      float best;
      int best_g;
      warp_argmax(gs, groups, lane, &best, &best_g);
      if (lane == 0) {
        gs[best_g] = -INFINITY;
        kept[best_g] = 1;
      }
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!kept[e / size]) c[e] = -INFINITY;  // struck out, not zero: choice scores can be negative
    __syncwarp();
  }
  float total = 0.f, mine = 0.f;
  int mine_e = 0;
  for (int j = 0; j < top; ++j) {
    float best;
    int best_e;
    warp_argmax(c, E, lane, &best, &best_e);
    const float v = s[best_e];
    total += v;
    if (lane == j) { mine = v; mine_e = best_e; }
    __syncwarp();
    if (lane == 0) c[best_e] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    experts[(size_t)row * top + lane] = mine_e;
    weights[(size_t)row * top + lane] = mine / (total + 1e-20f) * scale;
  }
}

constexpr int PAIR_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32)
moe_gate_up_pairs_kernel(T* __restrict__ act_out, const T* __restrict__ x, int x_stride, const T* __restrict__ w,
                         const int* __restrict__ experts, int top, int F, int K, int act) {
  extern __shared__ __align__(16) float xs[];  // [K]
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = blockIdx.y;
  const int e = experts[pair];
  const T* xr = x + (size_t)(pair / top) * x_stride;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float<T>(xr[k]);
  __syncthreads();
  const T* we = w + (size_t)e * 2 * F * K;
  for (int f = blockIdx.x * PAIR_WARPS + warp; f < F; f += gridDim.x * PAIR_WARPS) {
    const T* wg = we + (size_t)f * K;
    const T* wu = we + (size_t)(F + f) * K;
    const float g = warp_sum(lane_dot<T>(wg, xs, K, lane));
    const float u = warp_sum(lane_dot<T>(wu, xs, K, lane));
    // the two products leave in the path's type before the activation, as they do from a product kernel
    if (lane == 0) act_out[(size_t)pair * F + f] = from_float<T>(act_of(round_to<T>(g), act) * round_to<T>(u));
  }
}

template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32)
moe_down_pairs_kernel(T* __restrict__ out, const T* __restrict__ add, const float* __restrict__ add_gate, const T* __restrict__ act_in,
                      const T* __restrict__ w, const int* __restrict__ experts, const float* __restrict__ weights, int top,
                      int C, int F) {
  extern __shared__ __align__(16) float as[];  // [top][F4], F4 = F rounded up to a multiple of 4
  const int F4 = (F + 3) & ~3;
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.y;
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) as[(i / F) * F4 + i % F] = to_float<T>(act_in[(size_t)row * top * F + i]);
  __syncthreads();
  for (int c = blockIdx.x * PAIR_WARPS + warp; c < C; c += gridDim.x * PAIR_WARPS) {
    float total = add ? to_float<T>(add[(size_t)row * C + c]) * (add_gate ? add_gate[row] : 1.f) : 0.f;
    // four experts' rows are read side by side, so that four times the bytes are in flight; the results are still
    // added in the order of the choice
    for (int j0 = 0; j0 < top; j0 += 4) {
      const T* wr[4];
      float s[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = min(j0 + jj, top - 1);
        wr[jj] = w + ((size_t)experts[(size_t)row * top + j] * C + c) * F;
        s[jj] = 0.f;
      }
      if (sizeof(T) == 2 && (F & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        for (int k = lane * 8; k < F; k += 256) {
          uint4 raw[4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) raw[jj] = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(wr[jj]) + k);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float* xs = as + min(j0 + jj, top - 1) * F4 + k;
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[jj]);
            const float4 a = *reinterpret_cast<const float4*>(xs), b = *reinterpret_cast<const float4*>(xs + 4);
            s[jj] += __low2float(p[0]) * a.x + __high2float(p[0]) * a.y + __low2float(p[1]) * a.z + __high2float(p[1]) * a.w +
                     __low2float(p[2]) * b.x + __high2float(p[2]) * b.y + __low2float(p[3]) * b.z + __high2float(p[3]) * b.w;
          }
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) s[jj] = lane_dot<T>(wr[jj], as + min(j0 + jj, top - 1) * F4, F, lane);
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float r = warp_sum(s[jj]);
        if (j0 + jj < top) total += weights[(size_t)row * top + j0 + jj] * round_to<T>(r);
      }
    }
    if (lane == 0) out[(size_t)row * C + c] = from_float<T>(total);
  }
}

// One block: counts per expert, offsets, each pair's place in the expert order (stable: pairs of one expert
// keep their order), and the rows of x gathered in that order.
__global__ void moe_sort_kernel(int* __restrict__ offsets, int* __restrict__ place, const int* __restrict__ experts,
                                int pairs, int E) {
  extern __shared__ int cnt[];  // [E + 1]
  grid_dependency_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[experts[i] + 1], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < E; ++e) cnt[e + 1] += cnt[e];
    for (int e = 0; e <= E; ++e) offsets[e] = cnt[e];
  }
  __syncthreads();
  // a warp per expert walks the pairs in order, 32 at a time (a ballot gives each hit its rank): stable
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int e = warp; e < E; e += n_warps) {
    int at = cnt[e];
    for (int i0 = 0; i0 < pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < pairs && experts[i] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) place[i] = at + __popc(mask & ((1u << lane) - 1u));
      at += __popc(mask);
    }
  }
}

__device__ __forceinline__ int row_of_pair(const int* __restrict__ place, const int* __restrict__ experts,
                                           const int* __restrict__ offsets, int cap, int pair) {
  if (cap <= 0) return place[pair];
  const int e = experts[pair];
  return e * cap + place[pair] - offsets[e];
}

template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xg, const T* __restrict__ x, int x_stride, const int* __restrict__ place,
                                  const int* __restrict__ experts, const int* __restrict__ offsets, int cap, int top, int K) {
  grid_dependency_wait();
  const int pair = blockIdx.x;
  const T* src = x + (size_t)(pair / top) * x_stride;
  T* dst = xg + (size_t)row_of_pair(place, experts, offsets, cap, pair) * K;
  if ((K * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int n = K * (int)sizeof(T) / 16;
    for (int k = threadIdx.x; k < n; k += blockDim.x) reinterpret_cast<uint4*>(dst)[k] = reinterpret_cast<const uint4*>(src)[k];
    return;
  }
  for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = src[k];
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ add, const float* __restrict__ add_gate, const T* __restrict__ yg,
                                   const int* __restrict__ place, const int* __restrict__ experts,
                                   const int* __restrict__ offsets, int cap, const float* __restrict__ weights, int top,
                                   int C) {
  __shared__ int src_row[32];
  __shared__ float src_w[32];
  grid_dependency_wait();
  const int row = blockIdx.x;
  if (threadIdx.x < top) {
    src_row[threadIdx.x] = row_of_pair(place, experts, offsets, cap, row * top + threadIdx.x);
    src_w[threadIdx.x] = weights[(size_t)row * top + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float total = add ? to_float<T>(add[(size_t)row * C + c]) * (add_gate ? add_gate[row] : 1.f) : 0.f;
    for (int j = 0; j < top; ++j) total += src_w[j] * to_float<T>(yg[(size_t)src_row[j] * C + c]);
    out[(size_t)row * C + c] = from_float<T>(total);
  }
}

}  // namespace

KRK_API int krk_moe_route(int* experts, float* weights, float* row_gate, const float* logits, const float* bias, int rows,
                          int E, int has_gate, int top, cudaStream_t stream, int over_all) {
  if (rows == 0) return 0;
  if (top < 1 || top > 32 || top > E) return -2;
  const size_t smem = (size_t)ROUTE_WARPS * E * sizeof(float);
  if (smem > 48 * 1024) return -2;
  return (int)launch_pdl(moe_route_kernel, dim3((rows + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream,
                         experts, weights, row_gate, logits, bias, rows, E, has_gate, top, over_all);
}

KRK_API int krk_moe_route_groups(int* experts, float* weights, float* row_gate, const float* logits, const float* correction,
                                 int rows, int E, int has_gate, int top, int groups, int keep, float scale,
                                 cudaStream_t stream) {
  if (rows == 0) return 0;
  if (top < 1 || top > 32 || top > E || groups < 1 || E % groups || keep < 1 || keep > groups ||
      top > keep * (E / groups))
    return -2;
  const size_t smem = (size_t)ROUTE_WARPS * (2 * E + 2 * groups) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  return (int)launch_pdl(moe_route_groups_kernel, dim3((rows + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem,
                         stream, experts, weights, row_gate, logits, correction, rows, E, has_gate, top, groups, keep, scale);
}

KRK_API int krk_moe_gate_up_pairs(void* act_out, const void* x, int x_stride, const void* w, const int* experts, int rows,
                                  int top, int F, int K, int act, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  const size_t smem = (size_t)K * sizeof(float);
  if (smem > 200 * 1024 || (long long)rows * top > 65535) return -2;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(moe_gate_up_pairs_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(moe_gate_up_pairs_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const dim3 grid((unsigned)min((F + PAIR_WARPS - 1) / PAIR_WARPS, 1024), (unsigned)(rows * top));
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(moe_gate_up_pairs_kernel<float>, grid, dim3(PAIR_WARPS * 32), smem, stream, (float*)act_out,
                           (const float*)x, x_stride, (const float*)w, experts, top, F, K, act);
  return (int)launch_pdl(moe_gate_up_pairs_kernel<bf16>, grid, dim3(PAIR_WARPS * 32), smem, stream, (bf16*)act_out,
                         (const bf16*)x, x_stride, (const bf16*)w, experts, top, F, K, act);
}

KRK_API int krk_moe_down_pairs(void* out, const void* add, const float* add_gate, const void* act_in, const void* w, const int* experts,
                               const float* weights, int rows, int top, int C, int F, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  const size_t smem = (size_t)top * ((F + 3) & ~3) * sizeof(float);
  if (smem > 200 * 1024 || rows > 65535) return -2;
  if (smem > 48 * 1024) {  // many or wide experts a token: the block's copy of their activations needs the opt-in size
    cudaFuncSetAttribute(moe_down_pairs_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(moe_down_pairs_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const dim3 grid((unsigned)min((C + PAIR_WARPS - 1) / PAIR_WARPS, 1024), (unsigned)rows);
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(moe_down_pairs_kernel<float>, grid, dim3(PAIR_WARPS * 32), smem, stream, (float*)out,
                           (const float*)add, add_gate, (const float*)act_in, (const float*)w, experts, weights, top, C, F);
  return (int)launch_pdl(moe_down_pairs_kernel<bf16>, grid, dim3(PAIR_WARPS * 32), smem, stream, (bf16*)out,
                         (const bf16*)add, add_gate, (const bf16*)act_in, (const bf16*)w, experts, weights, top, C, F);
}

KRK_API int krk_moe_sort(int* offsets, int* place, const int* experts, int rows, int top, int E, cudaStream_t stream) {
  if (rows == 0) return 0;
  return (int)launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), stream, offsets, place,
                         experts, rows * top, E);
}

KRK_API int krk_moe_gather(void* xg, const void* x, int x_stride, const int* place, const int* experts, const int* offsets,
                           int cap, int rows, int top, int K, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  const int pairs = rows * top;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, stream, (float*)xg, (const float*)x,
                           x_stride, place, experts, offsets, cap, top, K);
  return (int)launch_pdl(moe_gather_kernel<bf16>, dim3(pairs), dim3(128), 0, stream, (bf16*)xg, (const bf16*)x, x_stride,
                         place, experts, offsets, cap, top, K);
}

KRK_API int krk_moe_combine(void* out, const void* add, const float* add_gate, const void* yg, const int* place, const int* experts,
                            const int* offsets, int cap, const float* weights, int rows, int top, int C, int dtype,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  if (top > 32) return -2;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(moe_combine_kernel<float>, dim3(rows), dim3(256), 0, stream, (float*)out, (const float*)add, add_gate,
                           (const float*)yg, place, experts, offsets, cap, weights, top, C);
  return (int)launch_pdl(moe_combine_kernel<bf16>, dim3(rows), dim3(256), 0, stream, (bf16*)out, (const bf16*)add, add_gate,
                         (const bf16*)yg, place, experts, offsets, cap, weights, top, C);
}
