// A state-space mixer with a matrix state per head and a scalar decay per head and token (Mamba-2).
//
// krk_causal_conv_silu: y[r, c] = silu(b[c] + sum_j w[j, c] * in[r - (taps - 1 - j), c]) over the rows of one
// sequence (the weights come tap-major, [taps, channels], so that a thread's channels lie side by side); rows before the step's first come from the sequence's stored tail (its last taps - 1 inputs),
// rows before the sequence's start are zero (the tail of a fresh slot is zero). krk_conv_tail_update then
// stores the new last taps - 1 inputs; it is a launch of its own because rows of the step still read the
// old tail while the step's last rows would overwrite it.
//
// krk_ssd_scan: per (sequence, head), with S [N, P] float32 carried from token to token,
//   dt = softplus(dt_raw + dt_bias_h);  a = exp(-exp(A_log_h) * dt)
//   S <- a S + dt B x^T;  y = S^T C + D_h x
// A block holds one head's state in registers: a group of one, two or four columns of S is spread over NS lanes
// of one warp, each holding a run of consecutive rows of those columns; a token's y_p is each lane's ordered
// partial sums followed by a fixed exchange between the NS lanes. Tokens are staged through shared memory sixteen
// at a time (x, B, C as float32, dt and a computed once per token), the next sixteen requested as asynchronous
// copies while these are computed. Steps of one sequence's many tokens run in three passes so that
// all SMs work on one sequence: every chunk of `chunk` tokens scans from a zero state to its local end state
// (pass 1), one small kernel walks a sequence's chunks in order, S_in[c+1] = (prod a) S_in[c] + local[c], and
// leaves every chunk its starting state and the sequence its final one (pass 2), and every chunk scans again
// from its starting state and writes y (pass 3). This regroups the sums of a state, nothing else.
//
// krk_gated_group_norm: v = y * silu(z); each of `parts` equal parts of the row is divided by its root mean
// square; times a weight and a scale; rounded once to the path's type.
#include "common.cuh"
#include "mma.cuh"  // cp.async

namespace {

constexpr int TOK = 16;       // tokens staged at a time
constexpr int MAX_TAPS = 16;  // the convolution's taps

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// V consecutive elements as floats, in one access of V * sizeof(T) bytes (the address is aligned to that)
template <typename T, int V> struct alignas(V * sizeof(T)) Run { T v[V]; };
template <typename T, int V> __device__ __forceinline__ void load_run(const T* p, float* f) {
  const Run<T, V> raw = *reinterpret_cast<const Run<T, V>*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) f[i] = to_float<T>(raw.v[i]);
}
template <typename T, int V> __device__ __forceinline__ void store_run(T* p, const float* f) {
  Run<T, V> raw;
#pragma unroll
  for (int i = 0; i < V; ++i) raw.v[i] = from_float<T>(f[i]);
  *reinterpret_cast<Run<T, V>*>(p) = raw;
}

// a thread takes V consecutive channels of one row (V = 1, or 16 bytes' worth where sizes and addresses allow)
template <typename T, int V>
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
  for (int c = V * (blockIdx.y * blockDim.x + threadIdx.x); c < ch; c += V * gridDim.y * blockDim.x) {
    constexpr int W = V >= 4 ? 4 : 1;  // the weights' floats in 16-byte pieces where the channels are (V = 1, 4 or 8)
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; i += W) load_run<float, W>(bias + c + i, acc + i);
    for (int j = 0; j < taps; ++j) {
      const int src = r - (keep - j);  // the row that tap j multiplies
      float v[V], wj[V];
      if (src >= first) load_run<T, V>(in + (size_t)src * in_stride + c, v);
      else load_run<T, V>(old + (size_t)(keep - (first - src)) * ch + c, v);  // first - src in 1..keep
#pragma unroll
      for (int i = 0; i < V; i += W) load_run<float, W>(w + (size_t)j * ch + c + i, wj + i);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += wj[i] * v[i];
    }
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = silu_f(acc[i]);
    store_run<T, V>(out + (size_t)r * ch + c, acc);
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
  int vec;               // x, B and C rows can be copied in 16-byte pieces (sizes, strides and addresses allow)
};

// MODE 0: the whole step of a sequence, from and to the stored state. MODE 1: a chunk from zero to its local
// end state (no y). MODE 3: a chunk from its starting state, y only.
// A lane holds NPT consecutive rows of PC consecutive columns of the state. NS lanes of one warp share a group of
// PC columns (lane ns holds rows n0 .. n0 + NPT - 1, n0 = ns * NPT); a warp covers PW = 32 / NS column groups, and
// lane = ns * PW + (group % PW), so that the lanes of one ns read one piece of B (or C) together. What a token
// costs a lane in shared-memory reads is 2 NPT + PC floats for 3 NPT PC multiply-adds, which is why a lane takes
// several columns where the state is large: the reads, not the arithmetic, bound the one-column form. B and C
// are staged with their rows padded with zeros up to NS * NPT, so that the token loop has no bounds to check
// (a row beyond N stays zero). Several columns a lane are taken only where P is a multiple of them, so that a
// lane's columns are one aligned piece of a row of x and of the state.
// y of a token: each lane's ordered partial sums over its rows, then over the NS lanes of the group: first
// log2(PC) exchange steps that halve the columns a lane carries while doubling the lanes summed into them, then
// plain exchanges; the order is fixed by (N, P) alone.
template <typename T, int NPT, int PC, int MODE>
__global__ void ssd_scan_kernel(SsdArgs a, int NS) {
  extern __shared__ __align__(16) float smem[];
  grid_launch_dependents();
  const int h = blockIdx.x, seq = blockIdx.y, chunk = MODE == 0 ? 0 : blockIdx.z;
  const int P = a.P, N = a.N, H = a.H;
  const int NP = NS * NPT;  // padded rows of B and C in shared memory
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int PW = 32 / NS;
  const int ns = lane / PW, p0 = (warp * PW + lane % PW) * PC;
  const int n0 = ns * NPT;
  constexpr int ACCS = PC == 1 ? 4 : (PC == 2 ? 2 : 1);  // ordered partial sums per column
  constexpr int LOG_PC = PC == 1 ? 0 : (PC == 2 ? 1 : 2);

  float* xs = smem;                 // [TOK][P]
  float* Bs = xs + TOK * P;         // [TOK][NP]
  float* Cs = Bs + TOK * NP;        // [TOK][NP]
  float* dts = Cs + TOK * NP;       // [TOK]
  float* as = dts + TOK;            // [TOK]
  float* ys = as + TOK;             // [TOK][P]
  for (int i = threadIdx.x; i < 2 * TOK * NP; i += blockDim.x) Bs[i] = 0.f;  // the padding stays zero
  const float bias = a.dt_bias[h], rate = expf(a.a_log[h]), skip = a.skip[h];  // weights: no kernel writes them

  grid_dependency_wait();
  const int qlen = a.seq_qlen[seq];
  const int t_lo = MODE == 0 ? 0 : chunk * a.chunk;
  if (t_lo >= qlen) return;
  const int t_hi = MODE == 0 ? qlen : min(qlen, t_lo + a.chunk);
  const int row0 = a.cu_q[seq];
  const int g = h / (H / a.G);

  float s[PC][NPT];
  float* st = nullptr;
  if (MODE == 0) st = a.state + ((size_t)a.seq_slot[seq] * H + h) * N * P;
  if (MODE == 3) st = a.chunk_state + (((size_t)seq * a.max_chunks + chunk) * H + h) * N * P;
  const bool live = p0 < P;  // with several columns a lane, P is a multiple of PC: all of them or none
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    float row[PC];
#pragma unroll
    for (int c = 0; c < PC; ++c) row[c] = 0.f;
    if (MODE != 1 && live && n0 + j < N) load_run<float, PC>(st + (size_t)(n0 + j) * P + p0, row);
#pragma unroll
    for (int c = 0; c < PC; ++c) s[c][j] = row[c];
  }
  float decay_prod = 1.f;

  // Where sizes and addresses allow, a tile's x, B and C rows come as asynchronous 16-byte copies into `raw`,
  // requested while the tile before is computed, and are widened from there into xs, Bs and Cs; a tile's dt
  // waits in a register of the thread that turns it into a step size and a decay.
  constexpr int V = 16 / (int)sizeof(T);
  T* raw = reinterpret_cast<T*>(ys + TOK * P);  // [TOK][P + 2 N]
  const int per_tok = P + 2 * N;
  const int ppt = (P + (MODE != 1 ? 2 : 1) * N) / V;  // pieces a token brings
  const bool vec = a.vec != 0;
  float dt_raw = 0.f;
  auto request = [&](int t0, int nt) {
    if (vec) {
      for (int i = threadIdx.x; i < nt * ppt; i += blockDim.x) {
        const int t = i / ppt, e = (i - t * ppt) * V;  // element e of the token's [x | B | C]
        const size_t r = (size_t)(row0 + t0 + t);
        const T* src = e < P ? (const T*)a.x + r * a.x_stride + h * P + e
                             : (e < P + N ? (const T*)a.B + r * a.b_stride + g * N + (e - P)
                                          : (const T*)a.C + r * a.c_stride + g * N + (e - P - N));
        cp_async_16(raw + t * per_tok + e, src);
      }
      cp_async_commit();
    }
    if (threadIdx.x < nt) dt_raw = to_float<T>(((const T*)a.dt)[(size_t)(row0 + t0 + threadIdx.x) * a.dt_stride + h]);
  };
  request(t_lo, min(TOK, t_hi - t_lo));

  for (int t0 = t_lo; t0 < t_hi; t0 += TOK) {
    const int nt = min(TOK, t_hi - t0);
    if (vec) cp_async_wait<0>();
    __syncthreads();  // the tile before is consumed (and its y stored); the first time: the padding is written
    if (vec) {
      for (int i = threadIdx.x; i < nt * ppt; i += blockDim.x) {
        const int t = i / ppt, e = (i - t * ppt) * V;
        float f[V];
        load_run<T, V>(raw + t * per_tok + e, f);
        float* dst = e < P ? xs + t * P + e : (e < P + N ? Bs + t * NP + (e - P) : Cs + t * NP + (e - P - N));
#pragma unroll
        for (int k = 0; k < V; k += 4) store_run<float, 4>(dst + k, f + k);
      }
    } else {
      for (int t = warp; t < nt; t += n_warps) {
        const size_t r = (size_t)(row0 + t0 + t);
        const T* xr = (const T*)a.x + r * a.x_stride + h * P;
        for (int c = lane; c < P; c += 32) xs[t * P + c] = to_float<T>(xr[c]);
        const T* br = (const T*)a.B + r * a.b_stride + g * N;
        for (int c = lane; c < N; c += 32) Bs[t * NP + c] = to_float<T>(br[c]);
        if (MODE != 1) {
          const T* cr = (const T*)a.C + r * a.c_stride + g * N;
          for (int c = lane; c < N; c += 32) Cs[t * NP + c] = to_float<T>(cr[c]);
        }
      }
    }
    if (threadIdx.x < nt) {
      const float d = softplus_f(dt_raw + bias);
      dts[threadIdx.x] = d;
      as[threadIdx.x] = expf(-rate * d);
    }
    __syncthreads();
    if (t0 + TOK < t_hi) request(t0 + TOK, min(TOK, t_hi - t0 - TOK));  // in flight while this tile is computed
    for (int t = 0; t < nt; ++t) {
      const float at = as[t], dtt = dts[t];
      float xv[PC], dx[PC], acc[PC][ACCS];
#pragma unroll
      for (int c = 0; c < PC; ++c) xv[c] = 0.f;
      if (live) load_run<float, PC>(xs + t * P + p0, xv);
#pragma unroll
      for (int c = 0; c < PC; ++c) {
        dx[c] = dtt * xv[c];
#pragma unroll
        for (int i = 0; i < ACCS; ++i) acc[c][i] = 0.f;
      }
      const float4* Bt = reinterpret_cast<const float4*>(Bs + t * NP + n0);
      const float4* Ct = reinterpret_cast<const float4*>(Cs + t * NP + n0);
#pragma unroll
      for (int j = 0; j < NPT / 4; ++j) {
        const float4 b4 = Bt[j];
        const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
        float cv[4] = {0.f, 0.f, 0.f, 0.f};
        if (MODE != 1) {
          const float4 c4 = Ct[j];
          cv[0] = c4.x; cv[1] = c4.y; cv[2] = c4.z; cv[3] = c4.w;
        }
#pragma unroll
        for (int c = 0; c < PC; ++c)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            s[c][4 * j + i] = fmaf(at, s[c][4 * j + i], bv[i] * dx[c]);
            if (MODE != 1) acc[c][i % ACCS] = fmaf(s[c][4 * j + i], cv[i], acc[c][i % ACCS]);
          }
      }
      if (MODE != 1) {
        float v[PC];
#pragma unroll
        for (int c = 0; c < PC; ++c)
          v[c] = ACCS == 4 ? (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]) : (ACCS == 2 ? acc[c][0] + acc[c][1] : acc[c][0]);
        int col = 0;
#pragma unroll
        for (int bit = 0; bit < LOG_PC; ++bit) {  // a lane gives half its columns to the lane that differs in this bit of ns
          const int half = PC >> (bit + 1);
          const bool up = (ns >> bit) & 1;
#pragma unroll
          for (int i = 0; i < half; ++i) {
            const float send = up ? v[i] : v[i + half];
            const float keep = up ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, PW << bit);
          }
          col += up ? half : 0;
        }
        for (int o = PW * PC; o < 32; o <<= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        if ((ns >> LOG_PC) == 0 && live) {
          float xc = xv[0];
#pragma unroll
          for (int c = 1; c < PC; ++c) xc = col == c ? xv[c] : xc;
          ys[t * P + p0 + col] = v[0] + skip * xc;
        }
      }
      if (MODE == 1) decay_prod *= at;
    }
    if (MODE != 1) {
      __syncthreads();
      for (int t = warp; t < nt; t += n_warps) {
        float* yr = a.y + (size_t)(row0 + t0 + t) * H * P + h * P;
        for (int c = lane; c < P; c += 32) yr[c] = ys[t * P + c];
      }
    }
  }
  if (MODE == 3) return;
  float* dst = MODE == 0 ? st : a.chunk_state + (((size_t)seq * a.max_chunks + chunk) * H + h) * N * P;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    float row[PC];
#pragma unroll
    for (int c = 0; c < PC; ++c) row[c] = s[c][j];
    if (live && n0 + j < N) store_run<float, PC>(dst + (size_t)(n0 + j) * P + p0, row);
  }
  if (MODE == 1 && threadIdx.x == 0) a.chunk_decay[((size_t)seq * a.max_chunks + chunk) * H + h] = decay_prod;
}

// pass 2: a sequence's chunks in order. chunk_state[c] holds chunk c's local end state and receives its
// starting state; the stored state receives the sequence's final one. The chunks' values are fetched eight at a
// time before the walk, which itself is a chain of dependent sums.
__global__ void ssd_combine_kernel(SsdArgs a) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int qlen = a.seq_qlen[seq];
  if (qlen <= 0) return;
  const int n_chunks = (qlen + a.chunk - 1) / a.chunk;
  const size_t NP = (size_t)a.N * a.P;
  float* st = a.state + ((size_t)a.seq_slot[seq] * a.H + h) * NP;
  const size_t step = (size_t)a.H * NP;  // from one chunk's state to the next one's
  for (size_t e = blockIdx.z * blockDim.x + threadIdx.x; e < NP; e += (size_t)gridDim.z * blockDim.x) {
    float run = st[e];
    float* cs = a.chunk_state + ((size_t)seq * a.max_chunks * a.H + h) * NP + e;
    const float* cd = a.chunk_decay + (size_t)seq * a.max_chunks * a.H + h;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {
      float local[8], decay[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + i < n_chunks) {
          local[i] = __ldcg(cs + (size_t)(c0 + i) * step);
          decay[i] = cd[(size_t)(c0 + i) * a.H];
        }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + i < n_chunks) {
          cs[(size_t)(c0 + i) * step] = run;
          run = fmaf(decay[i], run, local[i]);
        }
    }
    st[e] = run;
  }
}

template <typename T, int V>
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
  for (int i = V * threadIdx.x; i < n; i += V * blockDim.x) {
    float yv[V], zv[V];
    load_run<float, V>(y + (size_t)r * inner + c0 + i, yv);
    load_run<T, V>(z + (size_t)r * z_stride + c0 + i, zv);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float v = yv[k] * silu_f(zv[k]);
      row_s[i + k] = v;
      sq += v * v;
    }
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)n + eps);
  for (int i = V * threadIdx.x; i < n; i += V * blockDim.x) {
    float o[V];
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = row_s[i + k] * rstd * weight[c0 + i + k] * out_scale;
    store_run<T, V>(out + (size_t)r * out_stride + out_col + c0 + i, o);
  }
}

template <typename T, int MODE>
int launch_scan(const SsdArgs& a, int NS, int npt, int pc, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
#define KRK_SSD_CASE(V, C)                                                                                          \
  if (npt == V && pc == C) {                                                                                        \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(ssd_scan_kernel<T, V, C, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return (int)launch_pdl(ssd_scan_kernel<T, V, C, MODE>, grid, dim3(threads), smem, stream, a, NS);               \
  }
  KRK_SSD_CASE(4, 1)
  KRK_SSD_CASE(8, 1)
  KRK_SSD_CASE(16, 1)
  KRK_SSD_CASE(32, 1)
  KRK_SSD_CASE(64, 1)
  KRK_SSD_CASE(8, 2)
  KRK_SSD_CASE(8, 4)
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
  int npt = (N + NS - 1) / NS;
  if (npt > 64) return -2;
  npt = npt <= 4 ? 4 : npt <= 8 ? 8 : npt <= 16 ? 16 : npt <= 32 ? 32 : 64;  // the kernels' instantiations
  // a lane of 16 or 32 rows of one column becomes a lane of 8 rows of 2 or 4 columns (as many state elements
  // a lane, a half or a quarter of the reads of B and C a multiply-add)
  int pc = 1;
  if (npt == 16 && NS * 2 <= 32 && P % 2 == 0) { pc = 2; NS *= 2; npt = 8; }
  else if (npt == 32 && NS * 4 <= 32 && P % 4 == 0) { pc = 4; NS *= 4; npt = 8; }
  const int PW = 32 / NS;
  const int warps = (P + PW * pc - 1) / (PW * pc);
  if (warps > 32) return -2;
  const int threads = warps * 32;
  constexpr int V = 16 / (int)sizeof(T);
  a.vec = P % V == 0 && N % V == 0 && a.x_stride % V == 0 && a.b_stride % V == 0 && a.c_stride % V == 0 &&
          (((uintptr_t)a.x | (uintptr_t)a.B | (uintptr_t)a.C) & 15) == 0;
  const size_t smem = (size_t)(TOK * (2 * P + 2 * NS * npt) + 2 * TOK) * sizeof(float) +
                      (a.vec ? (size_t)TOK * (P + 2 * N) * sizeof(T) : 0);
  if (smem > 200 * 1024) return -2;
  if (a.chunk_state && a.chunk > 0 && max_q_len > a.chunk) {
    a.max_chunks = (max_q_len + a.chunk - 1) / a.chunk;
    dim3 grid(a.H, n_seqs, a.max_chunks);
    int rc = launch_scan<T, 1>(a, NS, npt, pc, grid, threads, smem, stream);
    if (rc) return rc;
    const int NP = N * P;
    rc = (int)launch_pdl(ssd_combine_kernel, dim3(a.H, n_seqs, (NP + 255) / 256), dim3(256), 0, stream, a);
    if (rc) return rc;
    return launch_scan<T, 3>(a, NS, npt, pc, grid, threads, smem, stream);
  }
  return launch_scan<T, 0>(a, NS, npt, pc, dim3(a.H, n_seqs), threads, smem, stream);
}

}  // namespace

KRK_API int krk_causal_conv_silu(void* out, const void* in, int in_stride, const float* w, const float* bias, void* tail,
                                 int taps, int ch, int rows, int n_seqs, const int* row_seq, const int* cu_q,
                                 const int* seq_qlen, const int* seq_slot, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return -2;
  const int threads = 256;
  const int cols = min(64, (ch + threads - 1) / threads);
  const int V = dtype == KRK_DTYPE_F32 ? 4 : 8;
  const bool vec = ch % V == 0 && in_stride % V == 0 &&
                   (((uintptr_t)in | (uintptr_t)out | (uintptr_t)tail | (uintptr_t)w | (uintptr_t)bias) & 15) == 0;
  const int vcols = min(64, (ch / V + threads - 1) / threads);
  int rc;
  if (dtype == KRK_DTYPE_F32) {
    auto kern = vec ? causal_conv_silu_kernel<float, 4> : causal_conv_silu_kernel<float, 1>;
    rc = (int)launch_pdl(kern, dim3(rows, vec ? vcols : cols), dim3(threads), 0, stream, (float*)out, (const float*)in,
                         in_stride, w, bias, (const float*)tail, taps, ch, row_seq, cu_q, seq_slot);
  } else {
    auto kern = vec ? causal_conv_silu_kernel<bf16, 8> : causal_conv_silu_kernel<bf16, 1>;
    rc = (int)launch_pdl(kern, dim3(rows, vec ? vcols : cols), dim3(threads), 0, stream, (bf16*)out, (const bf16*)in,
                         in_stride, w, bias, (const bf16*)tail, taps, ch, row_seq, cu_q, seq_slot);
  }
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
  a.chunk = chunk; a.max_chunks = 0; a.chunk_state = chunk_state; a.chunk_decay = chunk_decay; a.vec = 0;
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
  // four elements a thread (16 bytes of y, 8 or 16 of the gate and the result) where sizes and addresses allow
  const size_t esz = dtype == KRK_DTYPE_F32 ? 4 : 2;
  const bool vec = n % 4 == 0 && z_stride % 4 == 0 && out_stride % 4 == 0 && out_col % 4 == 0 &&
                   ((uintptr_t)y & 15) == 0 && (((uintptr_t)z | (uintptr_t)out) & (4 * esz - 1)) == 0;
  if (dtype == KRK_DTYPE_F32) {
    auto kern = vec ? gated_group_norm_kernel<float, 4> : gated_group_norm_kernel<float, 1>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)launch_pdl(kern, dim3(rows, parts), dim3(threads), smem, stream, (float*)out, out_stride, out_col,
                           out_scale, y, (const float*)z, z_stride, weight, inner, parts, eps);
  }
  auto kern = vec ? gated_group_norm_kernel<bf16, 4> : gated_group_norm_kernel<bf16, 1>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(rows, parts), dim3(threads), smem, stream, (bf16*)out, out_stride, out_col, out_scale,
                         y, (const bf16*)z, z_stride, weight, inner, parts, eps);
}
