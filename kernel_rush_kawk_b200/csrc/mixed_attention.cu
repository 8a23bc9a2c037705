// Attention whose heads' scores are mixed before the softmax, over the keys of the query's own block of
// positions, and the row kernels that a model built around it needs.
//
// krk_embed_bigram: x[r] = table[id_r] + pairs[(id_prev * a + id_r * b) mod m] (row m for a sequence's first token),
// float32 rows. id_prev of a step's first row is the sequence's stored last token; the block of that row reads it
// and then stores the step's last token in its place.
//
// krk_bias_norm_rotate_write: one warp per (row, head) of a stacked q | k | v product. Biases are added; a q or k
// head is divided by its root mean square and multiplied by a weight of the head's size (shared by the heads); the
// first `rot` elements are rotated by the position, element 2i with 2i + 1 (`pairs`) or i with i + rot/2; q is
// written back in place, k and v go to their pages. All arithmetic is float32 and a value is rounded once. The
// angle's sine and cosine are those of csrc/sink_attention.cu (frequencies as two floats each).
//
// krk_mixed_attention: one block per row, one warp per query head. The warps take 32 keys at a time, one key per
// lane: each lane's raw score is its own ordered sum over the head; the warps exchange their raw scores through
// shared memory and warp h forms s'_h = sum_g talk[h, g] s_g (g ascending); the softmax runs online with the sink
// as the starting state (maximum = sink, sum = 1, no value), and the float32 weights multiply the values with the
// lanes spread over the value head. A query at position p sees keys (p / chunk) * chunk .. p (chunk 0: 0 .. p). A
// row's result depends on that row's keys only, in their order: it is the same to the bit however the tokens were
// cut into steps or batched. Without `talk` no scores are exchanged.
//
// krk_mixed_attention_single (one token per sequence): the keys of a sequence are split over up to 32 blocks of a grid
// (split, sequence); every block does what the general kernel does over its share of the 32-key chunks and leaves
// (maximum, sum, output) per head; krk_mixed_attention_merge (one warp per (row, head), a lane per share for the
// maxima and sums) adds the shares in split order. The sink enters once, in the first split. The merge alone also
// serves the tensor-core prompt kernel where that deals a tile's pages out over several blocks.
//
// In both kernels a lane takes four consecutive elements of a value row as one piece per key, eight keys' pieces
// requested before the first is used, where the value head is a multiple of 4 up to 128 elements (else element
// lane + 32 i of every row), and a key row arrives four 16-byte pieces at a time.
//
// krk_norm_sum: out = scale * sum_b y_b / sqrt(mean(y_b^2) + eps) * gain_b over up to four inputs, float32 inside.
// krk_act_rows: an activation without a gate, elementwise (xIELU with its two slopes, tanh-GELU, SiLU).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ void angle_sincos2(float p, float f_hi, float f_lo, float* s, float* c) {
  const float a = __fmul_rn(p, f_hi);
  const float e = fmaf(p, f_hi, -a) + p * f_lo;
  float s0, c0;
  sincosf(a, &s0, &c0);
  *s = fmaf(e, c0, s0);
  *c = fmaf(-e, s0, c0);
}

template <typename T>
__global__ void embed_bigram_kernel(float* __restrict__ out, const T* __restrict__ table, const T* __restrict__ pairs,
                                    const int* __restrict__ ids, int* state, int H, int vocab, int buckets,
                                    long long mul_prev, long long mul_cur, const int* __restrict__ row_seq,
                                    const int* __restrict__ row_pos, const int* __restrict__ cu_q,
                                    const int* __restrict__ seq_slot, int* error) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int seq = row_seq[r];
  const int first_row = cu_q[seq];
  const int slot = seq_slot[seq];
  int id = ids[r];
  int prev = r == first_row ? state[slot] : ids[r - 1];
  const bool bad = id < 0 || id >= vocab || prev < 0 || prev >= vocab;
  if (bad) {
    if (threadIdx.x == 0 && error) atomicExch(error, 1);
    id = prev = 0;
  }
  const long long bucket = row_pos[r] == 0 ? (long long)buckets : (prev * mul_prev + id * mul_cur) % buckets;
  const T* a = table + (size_t)id * H;
  const T* b = pairs + (size_t)bucket * H;
  float* dst = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = bad ? 0.f : to_float<T>(a[i]) + to_float<T>(b[i]);
  if (r == first_row) {
    __syncthreads();  // every thread of this block has read the stored token
    if (threadIdx.x == 0) state[slot] = ids[cu_q[seq + 1] - 1];
  }
}

template <typename T>
__global__ void bias_norm_rotate_write_kernel(T* proj, int stride, int q_col, int k_col, int v_col, int HQ, int HKV, int D,
                                              int DV, const float* __restrict__ bias, const float* __restrict__ gain,
                                              float eps, const float* __restrict__ inv_freq, int rot, int pairs,
                                              const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                              const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                                              T* k_cache, T* v_cache, int rows, int keep_pages) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int per_row = HQ + 2 * HKV;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * per_row) return;
  const int row = (int)(item / per_row), which = (int)(item % per_row);
  const int pos = row_pos[row];
  T* base = proj + (size_t)row * stride;
  const T* src;
  T* dst;
  const float* b = bias;
  const float* g = nullptr;
  int n, turn;
  if (which < HQ) {
    src = dst = base + q_col + (size_t)which * D;
    if (b) b += (size_t)which * D;
    g = gain;
    n = D;
    turn = rot;
  } else {
    const int slot = seq_slot[row_seq[row]];
    const int page = page_of(table, width, slot, pos, keep_pages);
    if (which < HQ + HKV) {
      const int h = which - HQ;
      src = base + k_col + (size_t)h * D;
      dst = k_cache + (((size_t)page * HKV + h) * KRK_PAGE + (pos % KRK_PAGE)) * D;
      if (b) b += (size_t)HQ * D + (size_t)h * D;
      g = gain ? gain + D : nullptr;
      n = D;
      turn = rot;
    } else {
      const int h = which - HQ - HKV;
      src = base + v_col + (size_t)h * DV;
      dst = v_cache + (((size_t)page * HKV + h) * KRK_PAGE + (pos % KRK_PAGE)) * DV;
      if (b) b += (size_t)(HQ + HKV) * D + (size_t)h * DV;
      n = DV;
      turn = 0;
    }
  }
  float rstd = 1.f;
  if (g) {
    float sq = 0.f;
    for (int e = lane; e < n; e += 32) {
      const float x = to_float<T>(src[e]) + (b ? b[e] : 0.f);
      sq += x * x;
    }
    rstd = rsqrtf(warp_sum(sq) / (float)n + eps);
  }
  __syncwarp();  // q is rewritten in place: every lane has read what it needs of the head
  auto val = [&](int e) { return (to_float<T>(src[e]) + (b ? b[e] : 0.f)) * rstd * (g ? g[e] : 1.f); };
  const int half = turn >> 1;
  const float p = (float)pos;
  for (int i = lane; i < half; i += 32) {
    const int e0 = pairs ? 2 * i : i, e1 = pairs ? 2 * i + 1 : i + half;
    float s, c;
    angle_sincos2(p, inv_freq[i], inv_freq[half + i], &s, &c);
    const float u = val(e0), v = val(e1);
    dst[e0] = from_float<T>(u * c - v * s);
    dst[e1] = from_float<T>(v * c + u * s);
  }
  for (int e = turn + lane; e < n; e += 32) dst[e] = from_float<T>(val(e));
}

template <typename T> __device__ __forceinline__ float dot_key(const float* q, const T* k, int D) {
  float dot = 0.f;
  for (int d = 0; d < D; ++d) dot += q[d] * to_float<T>(k[d]);
  return dot;
}
// bfloat16 rows of a multiple of 8 elements start on 16-byte boundaries in the cache
template <> __device__ __forceinline__ float dot_key<bf16>(const float* q, const bf16* k, int D) {
  float dot = 0.f;
  if ((D & 7) == 0) {
    for (int d = 0; d < D; d += 32) {  // four 16-byte pieces are requested before the first is used
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (d + 8 * u < D) raw[u] = *reinterpret_cast<const uint4*>(k + d + 8 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (d + 8 * u < D) {
          const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            dot += q[d + 8 * u + 2 * j] * __low2float(p[j]);
            dot += q[d + 8 * u + 2 * j + 1] * __high2float(p[j]);
          }
        }
      }
    }
  } else {
    for (int d = 0; d < D; ++d) dot += q[d] * __bfloat162float(k[d]);
  }
  return dot;
}

// four consecutive elements of a value row (or zeros)
template <typename T> __device__ __forceinline__ void load4v(const T* p, float* f, bool on);
template <> __device__ __forceinline__ void load4v<float>(const float* p, float* f, bool on) {
  const float4 v = on ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4v<bf16>(const bf16* p, float* f, bool on) {
  const uint2 raw = on ? *reinterpret_cast<const uint2*>(p) : make_uint2(0u, 0u);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  f[0] = __low2float(h[0]); f[1] = __high2float(h[0]); f[2] = __low2float(h[1]); f[3] = __high2float(h[1]);
}

constexpr int MIX_VPL = 8;  // value heads up to 256

// The walk of one warp (= one query head of one row) over the 32-key chunks base = lo + 32 * (c0 + n * cstep), up to hi,
// together with the block's other warps. Leaves the running (m, l, acc). A lane's accumulators are elements lane + 32 i
// of the value head, or (V4: value heads of a multiple of 4 up to 128 elements) elements 4 lane .. 4 lane + 3, read
// as one piece per key, eight keys' pieces requested before the first is used.
template <typename T, bool V4>
__device__ __forceinline__ void mixed_walk(const float* qs, float* s_buf, const float* talk_s, int HQ, int HKV, int head,
                                           int D, int DV, int slot, int lo, int hi, int c0, int cstep,
                                           const int* __restrict__ table, int width, const T* __restrict__ k_cache,
                                           const T* __restrict__ v_cache, float scale, float& m, float& l, float* acc) {
  const int lane = threadIdx.x & 31;
  const int kh = head / (HQ / HKV);
  int it = 0;
  for (int base = lo + 32 * c0; base <= hi; base += 32 * cstep, ++it) {
    const int key = base + lane;
    const bool valid = key <= hi;
    float s = 0.f;
    int my_page = 0;
    if (valid) {
      my_page = page_of(table, width, slot, key);
      s = dot_key<T>(qs, k_cache + (((size_t)my_page * HKV + kh) * KRK_PAGE + (key % KRK_PAGE)) * D, D) * scale;
    }
    if (talk_s) {
      // two buffers in turn: a warp that runs ahead writes the other buffer, and cannot lap (one barrier a chunk)
      float* buf = s_buf + (size_t)(it & 1) * HQ * 32;
      buf[head * 32 + lane] = s;
      __syncthreads();
      float mixed = 0.f;
      for (int g = 0; g < HQ; ++g) mixed += talk_s[head * HQ + g] * buf[g * 32 + lane];
      s = mixed;
    }
    if (!valid) s = -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);  // exp(-inf) = 0 before the first key when there is no sink
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MIX_VPL; ++i) acc[i] *= alpha;
    const int n = min(32, hi - base + 1);
    if (V4) {
      const bool mine = 4 * lane < DV;
      for (int j0 = 0; j0 < n; j0 += 8) {
        float v[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = j0 + u;
          const int page = __shfl_sync(0xffffffffu, my_page, j & 31);  // lane j looked its key's page up already
          const T* vp = v_cache + (((size_t)page * HKV + kh) * KRK_PAGE + ((base + j) % KRK_PAGE)) * DV + 4 * lane;
          load4v<T>(vp, v[u], mine && j < n);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float pj = __shfl_sync(0xffffffffu, p, (j0 + u) & 31);  // 0 for a lane beyond the last key
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += pj * v[u][i];
        }
      }
    } else {
#pragma unroll 4
      for (int j = 0; j < n; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const int page = __shfl_sync(0xffffffffu, my_page, j);  // lane j looked its key's page up already
        const T* vp = v_cache + (((size_t)page * HKV + kh) * KRK_PAGE + ((base + j) % KRK_PAGE)) * DV;
#pragma unroll
        for (int i = 0; i < MIX_VPL; ++i) {
          const int d = lane + 32 * i;
          if (d < DV) acc[i] += pj * to_float<T>(vp[d]);
        }
      }
    }
    m = m_new;
  }
}

template <typename T, bool V4>
__global__ void mixed_attention_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                       const T* __restrict__ proj, int stride, int q_col, int HQ, int HKV, int D, int DV,
                                       const float* __restrict__ sink, const float* __restrict__ talk,
                                       const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                       const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                                       const T* __restrict__ k_cache, const T* __restrict__ v_cache, float scale, int chunk,
                                       const T* __restrict__ gate, int gate_stride, int gate_col, int gate_mode) {
  extern __shared__ __align__(16) float sm_mix[];
  float* q_s = sm_mix;                               // [HQ][D]
  float* s_buf = q_s + ((HQ * D + 3) & ~3);          // [2][HQ][32]
  float* talk_s = s_buf + 2 * HQ * 32;               // [HQ][HQ]
  if (talk)
    for (int i = threadIdx.x; i < HQ * HQ; i += blockDim.x) talk_s[i] = talk[i];  // weights: before the wait
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, head = threadIdx.x >> 5;
  const int row = blockIdx.x;
  const int pos = row_pos[row];
  const int slot = seq_slot[row_seq[row]];
  const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
  const T* q = proj + (size_t)row * stride + q_col;
  for (int i = threadIdx.x; i < HQ * D; i += blockDim.x) q_s[i] = to_float<T>(q[i]);
  __syncthreads();
  float m = sink ? sink[head] : -INFINITY;
  float l = sink ? 1.f : 0.f;
  float acc[MIX_VPL];
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) acc[i] = 0.f;
  mixed_walk<T, V4>(q_s + (size_t)head * D, s_buf, talk ? talk_s : nullptr, HQ, HKV, head, D, DV, slot, lo, pos, 0, 1, table,
                width, k_cache, v_cache, scale, m, l, acc);
  T* o = out + (size_t)row * out_stride + out_col + (size_t)head * DV;
  float inv = out_scale / l;
  if (gate_mode == 1) inv *= sigmoid_(to_float<T>(gate[(size_t)row * gate_stride + gate_col + head]));
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) {
    const int d = V4 ? 4 * lane + i : lane + 32 * i;
    if ((!V4 || i < 4) && d < DV) o[d] = from_float<T>(acc[i] * inv);
  }
}

// One token per sequence: block (split, sequence) takes every SPL-th 32-key chunk and leaves its share in
// scratch [seq][head][SPL][DV + 2] as (m, l, acc[DV]).
template <typename T, bool V4>
__global__ void mixed_attention_single_kernel(float* __restrict__ scratch, const T* __restrict__ proj, int stride, int q_col,
                                              int HQ, int HKV, int D, int DV, const float* __restrict__ sink,
                                              const float* __restrict__ talk, const int* __restrict__ seq_slot,
                                              const int* __restrict__ seq_start, const int* __restrict__ table, int width,
                                              const T* __restrict__ k_cache, const T* __restrict__ v_cache, float scale,
                                              int chunk, int SPL) {
  extern __shared__ __align__(16) float sm_mix[];
  float* q_s = sm_mix;
  float* s_buf = q_s + ((HQ * D + 3) & ~3);
  float* talk_s = s_buf + 2 * HQ * 32;
  if (talk)
    for (int i = threadIdx.x; i < HQ * HQ; i += blockDim.x) talk_s[i] = talk[i];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, head = threadIdx.x >> 5;
  const int split = blockIdx.x, seq = blockIdx.y;
  const int pos = seq_start[seq];  // the one new token sits at the sequence's length before the step
  const int slot = seq_slot[seq];
  const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
  const T* q = proj + (size_t)seq * stride + q_col;
  for (int i = threadIdx.x; i < HQ * D; i += blockDim.x) q_s[i] = to_float<T>(q[i]);
  __syncthreads();
  const bool with_sink = sink && split == 0;
  float m = with_sink ? sink[head] : -INFINITY;
  float l = with_sink ? 1.f : 0.f;
  float acc[MIX_VPL];
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) acc[i] = 0.f;
  mixed_walk<T, V4>(q_s + (size_t)head * D, s_buf, talk ? talk_s : nullptr, HQ, HKV, head, D, DV, slot, lo, pos, split, SPL,
                table, width, k_cache, v_cache, scale, m, l, acc);
  float* dst = scratch + (((size_t)seq * HQ + head) * SPL + split) * (DV + 2);
  if (lane == 0) {
    dst[0] = m;
    dst[1] = l;
  }
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) {
    const int d = V4 ? 4 * lane + i : lane + 32 * i;
    if ((!V4 || i < 4) && d < DV) dst[2 + d] = acc[i];
  }
}

// one warp per (sequence, head): the splits' shares in split order
template <typename T>
__global__ void mixed_attention_merge_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                             const float* __restrict__ scratch, int HQ, int DV, int SPL, int n_seqs,
                                             const T* __restrict__ gate, int gate_stride, int gate_col, int gate_mode) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_seqs * HQ) return;
  const int seq = item / HQ, head = item % HQ;
  const float* src = scratch + (size_t)item * SPL * (DV + 2);
  // lane s holds split s's maximum and sum (up to 32 splits); the outputs are added in split order
  const float my_m = lane < SPL ? src[(size_t)lane * (DV + 2)] : -INFINITY;
  const float my_l = lane < SPL ? src[(size_t)lane * (DV + 2) + 1] : 0.f;
  const float m = warp_max(my_m);
  const float my_w = lane < SPL ? expf(my_m - m) : 0.f;  // a split without keys left (-inf, 0, 0): weight 0
  const float l = warp_sum(my_w * my_l);
  float acc[MIX_VPL];
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) acc[i] = 0.f;
#pragma unroll 8
  for (int s = 0; s < SPL; ++s) {
    const float* p = src + (size_t)s * (DV + 2);
    const float w = __shfl_sync(0xffffffffu, my_w, s);
#pragma unroll
    for (int i = 0; i < MIX_VPL; ++i) {
      const int d = lane + 32 * i;
      if (d < DV) acc[i] += w * p[2 + d];
    }
  }
  float inv = out_scale / l;
  if (gate_mode == 1) inv *= sigmoid_(to_float<T>(gate[(size_t)seq * gate_stride + gate_col + head]));
  T* o = out + (size_t)seq * out_stride + out_col + (size_t)head * DV;
#pragma unroll
  for (int i = 0; i < MIX_VPL; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) o[d] = from_float<T>(acc[i] * inv);
  }
}

struct NormSumArgs {
  const void* y[4];
  const float* gain;  // [n][C]
  int n;
};

// V elements at a time (8 bfloat16 or 4 float32: 16 bytes); the row's inputs are held in shared memory between the
// sums of squares and the weighted sum, so that global memory is read once.
template <typename T, int V>
__global__ void norm_sum_kernel(T* __restrict__ out, NormSumArgs a, int C, float eps, float scale) {
  extern __shared__ __align__(16) float rows_s[];  // [n][C]
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t row = blockIdx.x;
  float sq[4] = {0.f, 0.f, 0.f, 0.f}, rstd[4];
  // all inputs' pieces are requested before any sum is formed
  for (int c = V * threadIdx.x; c < C; c += V * blockDim.x) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      if (b < a.n) {
        __align__(16) T raw[V];
        const T* y = reinterpret_cast<const T*>(a.y[b]) + row * C;
        if (V == 1) raw[0] = y[c];
        else *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(y + c);
        __align__(16) float f[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
          f[k] = to_float<T>(raw[k]);
          sq[b] += f[k] * f[k];
        }
        float* dst = rows_s + (size_t)b * C + c;
        if (V == 1) dst[0] = f[0];
        else
#pragma unroll
          for (int k = 0; k < V; k += 4) *reinterpret_cast<float4*>(dst + k) = *reinterpret_cast<const float4*>(f + k);
      }
    }
  }
  {  // the inputs' sums of squares through one exchange
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int b = 0; b < 4; ++b) sq[b] = warp_sum(sq[b]);
    if (lane == 0)
#pragma unroll
      for (int b = 0; b < 4; ++b) scratch[b * 8 + warp] = sq[b];
    __syncthreads();
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float t = 0.f;
      for (int w = 0; w < n_warps; ++w) t += scratch[b * 8 + w];
      rstd[b] = rsqrtf(t / (float)C + eps);
    }
  }
  for (int c = V * threadIdx.x; c < C; c += V * blockDim.x) {  // every thread reads back what it wrote
    __align__(16) T res[V];
    __align__(16) float total[V];
#pragma unroll
    for (int k = 0; k < V; ++k) total[k] = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      if (b >= a.n) break;
      __align__(16) float f[V], g[V];
      if (V == 1) {
        f[0] = rows_s[(size_t)b * C + c];
        g[0] = a.gain[(size_t)b * C + c];
      } else {
#pragma unroll
        for (int k = 0; k < V; k += 4) {
          *reinterpret_cast<float4*>(f + k) = *reinterpret_cast<const float4*>(rows_s + (size_t)b * C + c + k);
          *reinterpret_cast<float4*>(g + k) = *reinterpret_cast<const float4*>(a.gain + (size_t)b * C + c + k);
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) total[k] += f[k] * rstd[b] * g[k];
    }
#pragma unroll
    for (int k = 0; k < V; ++k) res[k] = from_float<T>(total[k] * scale);
    if (V == 1) out[row * C + c] = res[0];
    else *reinterpret_cast<uint4*>(out + row * C + c) = *reinterpret_cast<const uint4*>(res);
  }
}

__device__ __forceinline__ float act_value(float v, int act, float pa, float pb) {
  if (act == 4) return v > 0.f ? pa * v * v + 0.5f * v : pb * (expm1f(v) - v) + 0.5f * v;
  if (act == 1) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  return v / (1.0f + expf(-v));
}

// act 0: silu, 1: tanh-GELU, 4: xIELU with pa = softplus(p), pb = 1/2 + softplus(q). One block row (blockIdx.y) and
// column chunk; V elements (16 bytes) a thread at a time where the row allows it.
template <typename T, int V>
__global__ void act_rows_kernel(T* __restrict__ out, const T* __restrict__ z, int z_stride, int I, int act, float pa,
                                float pb) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t r = blockIdx.y;
  const T* src = z + r * z_stride;
  T* dst = out + r * I;
  for (int c = V * (blockIdx.x * blockDim.x + threadIdx.x); c < I; c += V * gridDim.x * blockDim.x) {
    __align__(16) T raw[V];
    __align__(16) T res[V];
    if (V == 1) raw[0] = src[c];
    else *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(src + c);
#pragma unroll
    for (int k = 0; k < V; ++k) res[k] = from_float<T>(act_value(to_float<T>(raw[k]), act, pa, pb));
    if (V == 1) dst[c] = res[0];
    else *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(res);
  }
}

size_t mixed_smem(int HQ, int D, bool talk) {
  return (size_t)(((HQ * D + 3) & ~3) + (talk ? 2 * HQ * 32 + HQ * HQ : 0)) * sizeof(float);
}

}  // namespace

KRK_API int krk_embed_bigram(float* out, const void* table, const void* pairs, const int* ids, int* state, int rows, int H,
                             int vocab, int buckets, long long mul_prev, long long mul_cur, const int* row_seq,
                             const int* row_pos, const int* cu_q, const int* seq_slot, int* error, int dtype,
                             cudaStream_t stream) {
  if (rows == 0) return 0;
  if (buckets < 1) return -2;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(embed_bigram_kernel<float>, dim3(rows), dim3(128), 0, stream, out, (const float*)table,
                           (const float*)pairs, ids, state, H, vocab, buckets, mul_prev, mul_cur, row_seq, row_pos, cu_q,
                           seq_slot, error);
  return (int)launch_pdl(embed_bigram_kernel<bf16>, dim3(rows), dim3(128), 0, stream, out, (const bf16*)table,
                         (const bf16*)pairs, ids, state, H, vocab, buckets, mul_prev, mul_cur, row_seq, row_pos, cu_q,
                         seq_slot, error);
}

KRK_API int krk_bias_norm_rotate_write(void* proj, int stride, int q_col, int k_col, int v_col, int HQ, int HKV, int D, int DV,
                                       const float* bias, const float* gain, float eps, const float* inv_freq, int rot,
                                       int pairs, const int* row_seq, const int* row_pos, const int* seq_slot,
                                       const int* table, int width, void* k_cache, void* v_cache, int rows, int keep_pages,
                                       int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rot < 0 || rot > D || (rot & 1)) return -2;
  const long long items = (long long)rows * (HQ + 2 * HKV);
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(bias_norm_rotate_write_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                           (float*)proj, stride, q_col, k_col, v_col, HQ, HKV, D, DV, bias, gain, eps, inv_freq, rot, pairs,
                           row_seq, row_pos, seq_slot, table, width, (float*)k_cache, (float*)v_cache, rows, keep_pages);
  return (int)launch_pdl(bias_norm_rotate_write_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                         (bf16*)proj, stride, q_col, k_col, v_col, HQ, HKV, D, DV, bias, gain, eps, inv_freq, rot, pairs,
                         row_seq, row_pos, seq_slot, table, width, (bf16*)k_cache, (bf16*)v_cache, rows, keep_pages);
}

KRK_API int krk_mixed_attention(void* out, int out_stride, int out_col, float out_scale, const void* proj, int stride,
                                int q_col, int HQ, int HKV, int D, int DV, const float* sink, const float* talk,
                                const int* row_seq, const int* row_pos, const int* seq_slot, const int* table, int width,
                                const void* k_cache, const void* v_cache, int rows, float scale, int chunk, const void* gate,
                                int gate_stride, int gate_col, int gate_mode, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (HQ < 1 || HQ > 32 || HKV < 1 || HQ % HKV || DV > 32 * MIX_VPL || gate_mode > 1 || chunk < 0) return -2;
  const size_t smem = mixed_smem(HQ, D, talk != nullptr);
  if (smem > 200 * 1024) return -2;
  const bool v4 = DV % 4 == 0 && DV <= 128;
  auto go = [&](auto kern, auto* tag) {
    typedef decltype(tag) P;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, dim3(rows), dim3(HQ * 32), smem, stream, (P)out, out_stride, out_col, out_scale, (P)proj,
                           stride, q_col, HQ, HKV, D, DV, sink, talk, row_seq, row_pos, seq_slot, table, width, (P)k_cache,
                           (P)v_cache, scale, chunk, (P)gate, gate_stride, gate_col, gate_mode);
  };
  if (dtype == KRK_DTYPE_F32)
    return v4 ? go(mixed_attention_kernel<float, true>, (float*)nullptr) : go(mixed_attention_kernel<float, false>, (float*)nullptr);
  return v4 ? go(mixed_attention_kernel<bf16, true>, (bf16*)nullptr) : go(mixed_attention_kernel<bf16, false>, (bf16*)nullptr);
}

// scratch: n_seqs * HQ * splits * (DV + 2) floats
KRK_API int krk_mixed_attention_single(void* out, int out_stride, int out_col, float out_scale, const void* proj, int stride,
                                       int q_col, int HQ, int HKV, int D, int DV, const float* sink, const float* talk,
                                       const int* seq_slot, const int* seq_start, const int* table, int width,
                                       const void* k_cache, const void* v_cache, int n_seqs, float scale, int chunk,
                                       int splits, float* scratch, const void* gate, int gate_stride, int gate_col,
                                       int gate_mode, int dtype, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (HQ < 1 || HQ > 32 || HKV < 1 || HQ % HKV || DV > 32 * MIX_VPL || gate_mode > 1 || chunk < 0 || splits < 1 ||
      splits > 32 || n_seqs > 65535)
    return -2;
  const size_t smem = mixed_smem(HQ, D, talk != nullptr);
  if (smem > 200 * 1024) return -2;
  const int merge_blocks = (n_seqs * HQ + 3) / 4;
  const bool v4 = DV % 4 == 0 && DV <= 128;
  auto go = [&](auto kern, auto merge, auto* tag) {
    typedef decltype(tag) P;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = launch_pdl(kern, dim3(splits, n_seqs), dim3(HQ * 32), smem, stream, scratch, (P)proj, stride, q_col, HQ, HKV,
                               D, DV, sink, talk, seq_slot, seq_start, table, width, (P)k_cache, (P)v_cache, scale, chunk,
                               splits);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(merge, dim3(merge_blocks), dim3(128), 0, stream, (decltype(tag))out, out_stride, out_col, out_scale,
                           (const float*)scratch, HQ, DV, splits, n_seqs, (P)gate, gate_stride, gate_col, gate_mode);
  };
  if (dtype == KRK_DTYPE_F32)
    return v4 ? go(mixed_attention_single_kernel<float, true>, mixed_attention_merge_kernel<float>, (float*)nullptr)
              : go(mixed_attention_single_kernel<float, false>, mixed_attention_merge_kernel<float>, (float*)nullptr);
  return v4 ? go(mixed_attention_single_kernel<bf16, true>, mixed_attention_merge_kernel<bf16>, (bf16*)nullptr)
            : go(mixed_attention_single_kernel<bf16, false>, mixed_attention_merge_kernel<bf16>, (bf16*)nullptr);
}

// The merge alone, for shares that another kernel left: items = rows of `out` (and of `gate`), scratch
// [items][HQ][splits][DV + 2] as (maximum, sum, output).
KRK_API int krk_mixed_attention_merge(void* out, int out_stride, int out_col, float out_scale, const float* scratch, int HQ,
                                      int DV, int splits, int items, const void* gate, int gate_stride, int gate_col,
                                      int gate_mode, int dtype, cudaStream_t stream) {
  if (items == 0) return 0;
  if (splits < 1 || splits > 32 || DV > 32 * MIX_VPL || gate_mode > 1) return -2;
  const long long blocks = ((long long)items * HQ + 3) / 4;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(mixed_attention_merge_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, (float*)out,
                           out_stride, out_col, out_scale, scratch, HQ, DV, splits, items, (const float*)gate, gate_stride,
                           gate_col, gate_mode);
  return (int)launch_pdl(mixed_attention_merge_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, (bf16*)out,
                         out_stride, out_col, out_scale, scratch, HQ, DV, splits, items, (const bf16*)gate, gate_stride,
                         gate_col, gate_mode);
}

KRK_API int krk_norm_sum(void* out, const void* y0, const void* y1, const void* y2, const void* y3, int n, const float* gain,
                         int rows, int C, float eps, float scale, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (n < 1 || n > 4) return -2;
  NormSumArgs a;
  a.y[0] = y0; a.y[1] = y1; a.y[2] = y2; a.y[3] = y3;
  a.gain = gain;
  a.n = n;
  const size_t smem = (size_t)n * C * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int V = dtype == KRK_DTYPE_F32 ? 4 : 8;
  const bool vec = C % V == 0 && (((uintptr_t)out | (uintptr_t)y0 | (uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)y3) & 15) == 0;
  const int pieces = vec ? C / V : C;
  const int threads = min(256, (pieces + 31) / 32 * 32);  // up to eight warps
  if (dtype == KRK_DTYPE_F32) {
    auto kern = vec ? norm_sum_kernel<float, 4> : norm_sum_kernel<float, 1>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (float*)out, a, C, eps, scale);
  }
  auto kern = vec ? norm_sum_kernel<bf16, 8> : norm_sum_kernel<bf16, 1>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(rows), dim3(threads), smem, stream, (bf16*)out, a, C, eps, scale);
}

KRK_API int krk_act_rows(void* out, const void* z, int z_stride, int rows, int I, int act, float pa, float pb, int dtype,
                         cudaStream_t stream) {
  if (rows == 0 || I == 0) return 0;
  if ((act != 0 && act != 1 && act != 4) || rows > 65535 * 16) return -2;
  const int V = dtype == KRK_DTYPE_F32 ? 4 : 8;
  const bool vec = I % V == 0 && z_stride % V == 0 && (((uintptr_t)out | (uintptr_t)z) & 15) == 0;
  const int pieces = vec ? I / V : I;
  const int chunks = min(64, (pieces + 255) / 256);
  // rows beyond a grid's second dimension are taken in slices
  const size_t esz = dtype == KRK_DTYPE_F32 ? 4 : 2;
  for (int r0 = 0; r0 < rows; r0 += 65535) {
    const int nr = min(65535, rows - r0);
    void* o = (char*)out + (size_t)r0 * I * esz;
    const void* src = (const char*)z + (size_t)r0 * z_stride * esz;
    cudaError_t e;
    if (dtype == KRK_DTYPE_F32)
      e = launch_pdl(vec ? act_rows_kernel<float, 4> : act_rows_kernel<float, 1>, dim3(chunks, nr), dim3(256), 0, stream,
                     (float*)o, (const float*)src, z_stride, I, act, pa, pb);
    else
      e = launch_pdl(vec ? act_rows_kernel<bf16, 8> : act_rows_kernel<bf16, 1>, dim3(chunks, nr), dim3(256), 0, stream,
                     (bf16*)o, (const bf16*)src, z_stride, I, act, pa, pb);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
