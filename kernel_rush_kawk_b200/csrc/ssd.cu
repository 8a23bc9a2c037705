// A state-space mixer with a matrix state per head and a scalar decay per head and token (Mamba-2).
//
// krk_causal_conv_silu: y[r, c] = silu(b[c] + sum_j w[c, j] * in[r - (taps - 1 - j), c]) over the rows of one
// sequence; rows before the step's first come from the sequence's stored tail (its last taps - 1 inputs),
// rows before the sequence's start are zero (the tail of a fresh slot is zero). krk_conv_tail_update then
// stores the new last taps - 1 inputs; it is a launch of its own because rows of the step still read the
// old tail while the step's last rows would overwrite it.
//
// krk_ssd_scan: per (sequence, head), with S [N, P] float32 carried from token to token,
//   dt = softplus(dt_raw + dt_bias_h);  a = exp(-exp(A_log_h) * dt)
//   S <- a S + dt B x^T;  y = S^T C + D_h x
// A block holds one head's state in registers: column p of S is spread over NS lanes of one warp, which hold
// the rows n = ns, ns + NS, ...; a token's y_p is each lane's ordered partial sum followed by a fixed
// exchange between the NS lanes. Tokens are staged through shared memory sixteen at a time (x, B, C as
// float32, dt and a computed once per token). Steps of one sequence's many tokens run in three passes so that
// all SMs work on one sequence: every chunk of `chunk` tokens scans from a zero state to its local end state
// (pass 1), one small kernel walks a sequence's chunks in order, S_in[c+1] = (prod a) S_in[c] + local[c], and
// leaves every chunk its starting state and the sequence its final one (pass 2), and every chunk scans again
// from its starting state and writes y (pass 3). This regroups the sums of a state, nothing else.
//
// krk_gated_group_norm: v = y * silu(z); each of `parts` equal parts of the row is divided by its root mean
// square; times a weight and a scale; rounded once to the path's type.
#include "common.cuh"

namespace {

constexpr int TOK = 16;       // tokens staged at a time
constexpr int MAX_TAPS = 16;  // the convolution's taps

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ in, int in_stride,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        const T* __restrict__ tail, int taps, int ch, const int* __restrict__ row_seq,
                                        const int* __restrict__ cu_q, const int* __restrict__ seq_slot) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int seq = row_seq[r];
  const int first = cu_q[seq];
  const int keep = taps - 1;
  const T* old = tail + (size_t)seq_slot[seq] * max(keep, 1) * ch;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ch; c += gridDim.y * blockDim.x) {
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {
      const int src = r - (keep - j);  // the row that column j multiplies
      float v;
      if (src >= first) v = to_float<T>(in[(size_t)src * in_stride + c]);
      else v = to_float<T>(old[(size_t)(keep - (first - src)) * ch + c]);  // first - src in 1..keep
      acc += w[(size_t)c * taps + j] * v;
    }
    out[(size_t)r * ch + c] = from_float<T>(silu_f(acc));
  }
}

// the sequence's last taps - 1 inputs after the step: from the step's rows, and from the old tail where the
// step brought fewer
template <typename T>
__global__ void conv_tail_update_kernel(T* tail, const T* __restrict__ in, int in_stride, int taps, int ch,
                                        const int* __restrict__ cu_q, const int* __restrict__ seq_qlen,
                                        const int* __restrict__ seq_slot) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int seq = blockIdx.x;
  const int keep = taps - 1;
  const int n = seq_qlen[seq], first = cu_q[seq];
  T* mine = tail + (size_t)seq_slot[seq] * keep * ch;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ch; c += gridDim.y * blockDim.x) {
    T v[MAX_TAPS];
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i) {
      if (i < keep) {
        const int back = keep - i;  // entry i is the input `back` tokens before the next token
        v[i] = back <= n ? in[(size_t)(first + n - back) * in_stride + c] : mine[(size_t)(i + n) * ch + c];
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_TAPS; ++i)
      if (i < keep) mine[(size_t)i * ch + c] = v[i];
  }
}

struct SsdArgs {
  const void *x, *B, *C, *dt;
  int x_stride, b_stride, c_stride, dt_stride;
  const float *dt_bias, *a_log, *skip;
  float* y;      // [rows, H * P]
  float* state;  // [slots, H, N, P]
  int H, P, N, G;
  const int *cu_q, *seq_qlen, *seq_slot;
  int chunk;             // tokens per chunk in the chunked passes
  int max_chunks;        // chunks of the longest sequence
  float* chunk_state;    // [n_seqs, max_chunks, H, N, P]
  float* chunk_decay;    // [n_seqs, max_chunks, H]
};

// MODE 0: the whole step of a sequence, from and to the stored state. MODE 1: a chunk from zero to its local
// end state (no y). MODE 3: a chunk from its starting state, y only.
template <typename T, int NPT, int MODE>
__global__ void ssd_scan_kernel(SsdArgs a, int NS) {
  extern __shared__ __align__(16) float smem[];
  grid_launch_dependents();
  grid_dependency_wait();
  const int h = blockIdx.x, seq = blockIdx.y, chunk = MODE == 0 ? 0 : blockIdx.z;
  const int P = a.P, N = a.N, H = a.H;
  const int qlen = a.seq_qlen[seq];
  const int t_lo = MODE == 0 ? 0 : chunk * a.chunk;
  if (t_lo >= qlen) return;
  const int t_hi = MODE == 0 ? qlen : min(qlen, t_lo + a.chunk);
  const int row0 = a.cu_q[seq];
  const int g = h / (H / a.G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int PW = 32 / NS;
  const int ns = lane / PW, p = warp * PW + lane % PW;
  const bool live = p < P;

  float* xs = smem;                 // [TOK][P]
  float* Bs = xs + TOK * P;         // [TOK][N]
  float* Cs = Bs + TOK * N;         // [TOK][N]
  float* dts = Cs + TOK * N;        // [TOK]
  float* as = dts + TOK;            // [TOK]
  float* ys = as + TOK;             // [TOK][P]

  float s[NPT];
  float* st = nullptr;
  if (MODE == 0) st = a.state + ((size_t)a.seq_slot[seq] * H + h) * N * P;
  if (MODE == 3) st = a.chunk_state + (((size_t)seq * a.max_chunks + chunk) * H + h) * N * P;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    const int n = ns + j * NS;
    s[j] = (MODE != 1 && live && n < N) ? st[(size_t)n * P + p] : 0.f;
  }
  const float bias = a.dt_bias[h], rate = expf(a.a_log[h]), skip = a.skip[h];
  float decay_prod = 1.f;

  for (int t0 = t_lo; t0 < t_hi; t0 += TOK) {
    const int nt = min(TOK, t_hi - t0);
    __syncthreads();  // the tile before is consumed (and its y stored)
    for (int i = threadIdx.x; i < nt * P; i += blockDim.x) {
      const int t = i / P, c = i % P;
      xs[t * P + c] = to_float<T>(((const T*)a.x)[(size_t)(row0 + t0 + t) * a.x_stride + h * P + c]);
    }
    for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
      const int t = i / N, c = i % N;
      Bs[t * N + c] = to_float<T>(((const T*)a.B)[(size_t)(row0 + t0 + t) * a.b_stride + g * N + c]);
      if (MODE != 1) Cs[t * N + c] = to_float<T>(((const T*)a.C)[(size_t)(row0 + t0 + t) * a.c_stride + g * N + c]);
    }
    if (threadIdx.x < nt) {
      const float d = softplus_f(to_float<T>(((const T*)a.dt)[(size_t)(row0 + t0 + threadIdx.x) * a.dt_stride + h]) + bias);
      dts[threadIdx.x] = d;
      as[threadIdx.x] = expf(-rate * d);
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float at = as[t];
      const float xv = live ? xs[t * P + p] : 0.f;
      const float dx = dts[t] * xv;
      const float* Bt = Bs + t * N;
      const float* Ct = Cs + t * N;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NPT; ++j) {
        const int n = ns + j * NS;
        if (n < N) {
          s[j] = at * s[j] + Bt[n] * dx;
          if (MODE != 1) acc += s[j] * Ct[n];
        }
      }
      if (MODE != 1) {
        for (int o = PW; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (ns == 0 && live) ys[t * P + p] = acc + skip * xv;
      }
      if (MODE == 1) decay_prod *= at;
    }
    if (MODE != 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < nt * P; i += blockDim.x) {
        const int t = i / P, c = i % P;
        a.y[(size_t)(row0 + t0 + t) * H * P + h * P + c] = ys[t * P + c];
      }
    }
  }
  if (MODE == 3) return;
  float* dst = MODE == 0 ? st : a.chunk_state + (((size_t)seq * a.max_chunks + chunk) * H + h) * N * P;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    const int n = ns + j * NS;
    if (live && n < N) dst[(size_t)n * P + p] = s[j];
  }
  if (MODE == 1 && threadIdx.x == 0) a.chunk_decay[((size_t)seq * a.max_chunks + chunk) * H + h] = decay_prod;
}

// pass 2: a sequence's chunks in order. chunk_state[c] holds chunk c's local end state and receives its
// starting state; the stored state receives the sequence's final one.
__global__ void ssd_combine_kernel(SsdArgs a) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int qlen = a.seq_qlen[seq];
  if (qlen <= 0) return;
  const int n_chunks = (qlen + a.chunk - 1) / a.chunk;
  const size_t NP = (size_t)a.N * a.P;
  float* st = a.state + ((size_t)a.seq_slot[seq] * a.H + h) * NP;
  for (size_t e = blockIdx.z * blockDim.x + threadIdx.x; e < NP; e += (size_t)gridDim.z * blockDim.x) {
    float run = st[e];
    for (int c = 0; c < n_chunks; ++c) {
      const size_t at = ((size_t)seq * a.max_chunks + c) * a.H + h;
      float* cs = a.chunk_state + at * NP + e;
      const float local = *cs;
      *cs = run;
      run = a.chunk_decay[at] * run + local;
    }
    st[e] = run;
  }
}

template <typename T>
__global__ void gated_group_norm_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                        const float* __restrict__ y, const T* __restrict__ z, int z_stride,
                                        const float* __restrict__ weight, int inner, int parts, float eps) {
  extern __shared__ __align__(16) float row_s[];  // one part of the row
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x, part = blockIdx.y;
  const int n = inner / parts, c0 = part * n;
  float sq = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = y[(size_t)r * inner + c0 + i] * silu_f(to_float<T>(z[(size_t)r * z_stride + c0 + i]));
    row_s[i] = v;
    sq += v * v;
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[(size_t)r * out_stride + out_col + c0 + i] = from_float<T>(row_s[i] * rstd * weight[c0 + i] * out_scale);
}

template <typename T, int MODE>
int launch_scan(const SsdArgs& a, int NS, int npt, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
#define KRK_SSD_CASE(V)                                                                                          \
  if (npt <= V) {                                                                                                \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(ssd_scan_kernel<T, V, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return (int)launch_pdl(ssd_scan_kernel<T, V, MODE>, grid, dim3(threads), smem, stream, a, NS);               \
  }
  KRK_SSD_CASE(4)
  KRK_SSD_CASE(8)
  KRK_SSD_CASE(16)
  KRK_SSD_CASE(32)
  KRK_SSD_CASE(64)
#undef KRK_SSD_CASE
  return -2;
}

template <typename T>
int run_scan(SsdArgs a, int n_seqs, int max_q_len, cudaStream_t stream) {
  const int P = a.P, N = a.N;
  // lanes per column: enough for 128 threads a block, and more while a lane would hold over 32 rows
  int NS = 1;
  while (NS < 32 && P * NS < 128) NS <<= 1;
  while (NS < 32 && (N + NS - 1) / NS > 32 && P * NS * 2 <= 1024) NS <<= 1;
  const int PW = 32 / NS;
  const int warps = (P + PW - 1) / PW;
  if (warps > 32) return -2;
  const int npt = (N + NS - 1) / NS;
  if (npt > 64) return -2;
  const int threads = warps * 32;
  const size_t smem = (size_t)(TOK * (2 * P + 2 * N) + 2 * TOK) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (a.chunk_state && a.chunk > 0 && max_q_len > a.chunk) {
    a.max_chunks = (max_q_len + a.chunk - 1) / a.chunk;
    dim3 grid(a.H, n_seqs, a.max_chunks);
    int rc = launch_scan<T, 1>(a, NS, npt, grid, threads, smem, stream);
    if (rc) return rc;
    const int NP = N * P;
    rc = (int)launch_pdl(ssd_combine_kernel, dim3(a.H, n_seqs, (NP + 1023) / 1024), dim3(256), 0, stream, a);
    if (rc) return rc;
    return launch_scan<T, 3>(a, NS, npt, grid, threads, smem, stream);
  }
  return launch_scan<T, 0>(a, NS, npt, dim3(a.H, n_seqs), threads, smem, stream);
}

}  // namespace

KRK_API int krk_causal_conv_silu(void* out, const void* in, int in_stride, const float* w, const float* bias, void* tail,
                                 int taps, int ch, int rows, int n_seqs, const int* row_seq, const int* cu_q,
                                 const int* seq_qlen, const int* seq_slot, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return -2;
  const int threads = 256;
  const int cols = min(64, (ch + threads - 1) / threads);
  int rc;
  if (dtype == KRK_DTYPE_F32)
    rc = (int)launch_pdl(causal_conv_silu_kernel<float>, dim3(rows, cols), dim3(threads), 0, stream, (float*)out,
                         (const float*)in, in_stride, w, bias, (const float*)tail, taps, ch, row_seq, cu_q, seq_slot);
  else
    rc = (int)launch_pdl(causal_conv_silu_kernel<bf16>, dim3(rows, cols), dim3(threads), 0, stream, (bf16*)out,
                         (const bf16*)in, in_stride, w, bias, (const bf16*)tail, taps, ch, row_seq, cu_q, seq_slot);
  if (rc || taps == 1) return rc;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(conv_tail_update_kernel<float>, dim3(n_seqs, cols), dim3(threads), 0, stream, (float*)tail,
                           (const float*)in, in_stride, taps, ch, cu_q, seq_qlen, seq_slot);
  return (int)launch_pdl(conv_tail_update_kernel<bf16>, dim3(n_seqs, cols), dim3(threads), 0, stream, (bf16*)tail,
                         (const bf16*)in, in_stride, taps, ch, cu_q, seq_qlen, seq_slot);
}

KRK_API int krk_ssd_scan(float* y, const void* x, int x_stride, const void* B, int b_stride, const void* C, int c_stride,
                         const void* dt, int dt_stride, const float* dt_bias, const float* a_log, const float* skip,
                         float* state, int H, int P, int N, int G, int n_seqs, int max_q_len, const int* cu_q,
                         const int* seq_qlen, const int* seq_slot, int chunk, float* chunk_state, float* chunk_decay,
                         int dtype, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (H % G) return -2;
  SsdArgs a;
  a.x = x; a.B = B; a.C = C; a.dt = dt;
  a.x_stride = x_stride; a.b_stride = b_stride; a.c_stride = c_stride; a.dt_stride = dt_stride;
  a.dt_bias = dt_bias; a.a_log = a_log; a.skip = skip; a.y = y; a.state = state;
  a.H = H; a.P = P; a.N = N; a.G = G;
  a.cu_q = cu_q; a.seq_qlen = seq_qlen; a.seq_slot = seq_slot;
  a.chunk = chunk; a.max_chunks = 0; a.chunk_state = chunk_state; a.chunk_decay = chunk_decay;
  return dtype == KRK_DTYPE_F32 ? run_scan<float>(a, n_seqs, max_q_len, stream) : run_scan<bf16>(a, n_seqs, max_q_len, stream);
}

KRK_API int krk_gated_group_norm(void* out, int out_stride, int out_col, float out_scale, const float* y, const void* z,
                                 int z_stride, const float* weight, int rows, int inner, int parts, float eps, int dtype,
                                 cudaStream_t stream) {
  if (rows == 0) return 0;
  if (parts < 1 || inner % parts) return -2;
  const int n = inner / parts;
  const size_t smem = (size_t)n * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  if (dtype == KRK_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_group_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(gated_group_norm_kernel<float>, dim3(rows, parts), dim3(threads), smem, stream, (float*)out,
                           out_stride, out_col, out_scale, y, (const float*)z, z_stride, weight, inner, parts, eps);
  }
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(gated_group_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(gated_group_norm_kernel<bf16>, dim3(rows, parts), dim3(threads), smem, stream, (bf16*)out,
                         out_stride, out_col, out_scale, y, (const bf16*)z, z_stride, weight, inner, parts, eps);
}
