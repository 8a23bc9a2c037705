// Mixers with a matrix-valued recurrent state per head: the token shift of RWKV-style time
// mixing, and one scan kernel for two update rules.
//
// State S [N key channels, N value channels] per (sequence, head), float32, in global memory
// between steps. With r, k, v of a token, a decay w and (delta rule) a removal rate a:
//
//   rule 0 (WKV):    o = (S + diag(bonus) k v^T)^T r ;  S <- diag(w) S + k v^T
//   rule 1 (delta):  u = k / sqrt(sum k^2 + 1e-6) ;  S <- diag(w) S - (a * u)(u^T S) + k v^T ;  o = S^T r
//
//   z = W2 tanh(lora) + w0 ;  w = exp(-exp(z)) (rule 0)  or  exp(-decay_scale * sigmoid(z)) (rule 1)
//   a = sigmoid(rate + rate_bias)
//   out = o / sqrt(mean_head(o^2) + eps) * norm_w * gate(g) * out_scale, gate = silu (rule 0) or sigmoid (rule 1)
//
// One block per (sequence, head). Column j of S (all key channels of one value channel) is spread over
// KL adjacent lanes, 16 or 32 key channels each, in registers for the whole pass; a sum over key channels
// is each lane's ordered partial sum followed by a fixed exchange between the KL lanes, and the token
// loop has no block-wide barrier. Tokens are taken in chunks, and the block is two groups of threads:
// while one scans a chunk, the other computes the next chunk's decays, unit keys and rates into shared
// memory (float32) and normalises, gates and stores the chunk before. A token's result is the same to
// the bit however the sequence was cut into steps: the chunking regroups work, not sums.
#include "mma.cuh"  // cp.async

namespace {

// out[s, r, c] = h[r, c] + (prev[r, c] - h[r, c]) * mu[s, c]; prev is the row before, or the
// sequence's stored last row for the first row of its step. With `store`, the thread that read element c of the
// stored row then puts element c of the step's last row of that sequence in its place.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const T* __restrict__ h, int h_stride, float* last_state,
                                   const float* __restrict__ mu, int n_mix, int C, int rows,
                                   const int* __restrict__ row_seq, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_slot, int store) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int seq = row_seq[r];
  const bool first = cu_q[seq] == r;
  float* last = last_state + (size_t)seq_slot[seq] * C;
  const int last_row = cu_q[seq + 1] - 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float hv = to_float<T>(h[(size_t)r * h_stride + c]);
    const float pv = first ? last[c] : to_float<T>(h[(size_t)(r - 1) * h_stride + c]);
    if (first && store) last[c] = to_float<T>(h[(size_t)last_row * h_stride + c]);
    const float d = pv - hv;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * rows + r) * C + c] = from_float<T>(hv + d * mu[(size_t)s * C + c]);
  }
}

struct ScanArgs {
  const void *r, *k, *v, *g, *rate, *lora;
  int r_stride, k_stride, v_stride, g_stride, rate_stride, lora_stride;
  const void* w2;          // [H*N, R], element type of the path
  const float* w0;         // [H*N]
  const float* rate_bias;  // [H*N] (rule 1)
  const float* bonus;      // [H*N] (rule 0)
  const float* norm_w;     // [H*N]
  float* state;            // [slots, H, N, N]
  const void* last_rows;   // rows whose last one per sequence is stored (rule 0's token shift), or null
  int last_stride, C;
  float* last_state;       // [slots, C]
  void* out;
  int out_stride, out_col;
  float out_scale, eps, decay_scale;
  int H, N, R, n_seqs;
  const int *cu_q, *seq_qlen, *seq_slot;
  int vec;  // rows, strides and the head size allow accesses of four elements at a time
};

template <typename T> __device__ __forceinline__ void load4_el(const T* p, float* f);
template <> __device__ __forceinline__ void load4_el<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4_el<bf16>(const bf16* p, float* f) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  f[0] = __low2float(h[0]); f[1] = __high2float(h[0]); f[2] = __low2float(h[1]); f[3] = __high2float(h[1]);
}
template <typename T> __device__ __forceinline__ void store4_el(T* p, const float* f);
template <> __device__ __forceinline__ void store4_el<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4_el<bf16>(bf16* p, const float* f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

// CPT: columns of S per scanning thread (every staged vector it reads serves all of them).

// One token's update of a thread's share of the state (CPT columns x NPT key channels) and its outputs,
// summed over the KL lanes of a column. Both scan kernels run exactly this, so a token's result does not
// depend on which of them served its step.
template <int RULE, int NPT, int CPT>
__device__ __forceinline__ void scan_token(float (&S)[CPT][NPT], const float4* r4, const float4* k4, const float4* w4,
                                           const float4* u4, const float4* a4, const float (&vj)[CPT], int KL,
                                           float (&o)[CPT]) {
  float o0[CPT], o1[CPT];
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2) o0[c2] = o1[c2] = 0.f;
  if (RULE == 1) {
    float s0[CPT], s1[CPT], uS[CPT];
#pragma unroll
    for (int c2 = 0; c2 < CPT; ++c2) s0[c2] = s1[c2] = 0.f;
#pragma unroll
    for (int q = 0; q < NPT / 4; ++q) {
      const float4 u = u4[q];
#pragma unroll
      for (int c2 = 0; c2 < CPT; ++c2) {
        s0[c2] += u.x * S[c2][4 * q];
        s1[c2] += u.y * S[c2][4 * q + 1];
        s0[c2] += u.z * S[c2][4 * q + 2];
        s1[c2] += u.w * S[c2][4 * q + 3];
      }
    }
#pragma unroll
    for (int c2 = 0; c2 < CPT; ++c2) {
      uS[c2] = s0[c2] + s1[c2];
      for (int off = 1; off < KL; off <<= 1) uS[c2] += __shfl_xor_sync(0xffffffffu, uS[c2], off);
    }
#pragma unroll
    for (int q = 0; q < NPT / 4; ++q) {
      const float4 w = w4[q], au = a4[q], k = k4[q], r = r4[q];
#pragma unroll
      for (int c2 = 0; c2 < CPT; ++c2) {
        float* Sc = S[c2];
        Sc[4 * q] = w.x * Sc[4 * q] - au.x * uS[c2] + k.x * vj[c2];
        o0[c2] += r.x * Sc[4 * q];
        Sc[4 * q + 1] = w.y * Sc[4 * q + 1] - au.y * uS[c2] + k.y * vj[c2];
        o1[c2] += r.y * Sc[4 * q + 1];
        Sc[4 * q + 2] = w.z * Sc[4 * q + 2] - au.z * uS[c2] + k.z * vj[c2];
        o0[c2] += r.z * Sc[4 * q + 2];
        Sc[4 * q + 3] = w.w * Sc[4 * q + 3] - au.w * uS[c2] + k.w * vj[c2];
        o1[c2] += r.w * Sc[4 * q + 3];
      }
    }
  } else {
#pragma unroll
    for (int q = 0; q < NPT / 4; ++q) {
      const float4 w = w4[q], u = u4[q], k = k4[q], r = r4[q];
#pragma unroll
      for (int c2 = 0; c2 < CPT; ++c2) {
        float* Sc = S[c2];
        o0[c2] += r.x * (Sc[4 * q] + u.x * vj[c2]);
        Sc[4 * q] = w.x * Sc[4 * q] + k.x * vj[c2];
        o1[c2] += r.y * (Sc[4 * q + 1] + u.y * vj[c2]);
        Sc[4 * q + 1] = w.y * Sc[4 * q + 1] + k.y * vj[c2];
        o0[c2] += r.z * (Sc[4 * q + 2] + u.z * vj[c2]);
        Sc[4 * q + 2] = w.z * Sc[4 * q + 2] + k.z * vj[c2];
        o1[c2] += r.w * (Sc[4 * q + 3] + u.w * vj[c2]);
        Sc[4 * q + 3] = w.w * Sc[4 * q + 3] + k.w * vj[c2];
      }
    }
  }
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2) {
    o[c2] = o0[c2] + o1[c2];
    for (int off = 1; off < KL; off <<= 1) o[c2] += __shfl_xor_sync(0xffffffffu, o[c2], off);
  }
}

template <int PROD>
__device__ __forceinline__ void producers_sync_n() { asm volatile("bar.sync 1, %0;" ::"n"(PROD) : "memory"); }

// NPT: key channels of a column that one lane keeps (16 for heads of up to 64 channels, 32 up to 128), CPT = 2
// columns a thread. Lighter threads (8 channels, one column: four times the warps) were measured and are slower,
// 0.83 against 0.60 us a token: every warp reads every staged vector, and shared-memory loads and the lanes'
// exchanges, not issue slots, then bound the scan.
// A lane's slice of a staged vector starts NPT + 4 floats after its neighbour's, so that the four
// slices a quarter-warp reads at once fall into different banks. TC: tokens per chunk.
//
// The block's first `cons` threads scan; its last PROD threads (a multiple of 32) prepare the chunk after the one being
// scanned (stage r, k, v; unit-key norms; decays and rates) into the other of two buffers and finish the
// chunk before it (per-head norm, weight, gate, store). The two groups meet once per chunk.
template <typename T, int RULE, int NPT, int CPT, int TC, int PROD, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) recurrence_kernel(ScanArgs a, int KL, int cons) {
  constexpr int SL = NPT + 4;
  auto producers_sync = [] { producers_sync_n<PROD>(); };
  extern __shared__ __align__(16) float sm[];
  const int N = a.N, R = a.R;
  const int VS = KL * SL;            // floats of one staged vector of one token
  const int BUF = 5 * TC * VS + TC * N;  // r, k, decay, u, au (padded slices), then v [TC][N]
  float* o_s = sm + 2 * BUF;         // [2][TC][N]
  float* w2_s = o_s + 2 * TC * N;    // [R][N]
  float* th_s = w2_s + R * N;        // [TC][R] tanh of the low-rank input
  float* red_s = th_s + TC * R;      // [2][TC] per-token reductions of the producers

  grid_launch_dependents();
  const int seq = blockIdx.x / a.H, head = blockIdx.x % a.H;
  const int tid = threadIdx.x;
  const int ch0 = head * N;
  // weights first (no kernel writes them), and zeros where a slice reaches past the head's channels
  for (int i = tid; i < R * N; i += blockDim.x) {
    const int m = i / N, c = i % N;
    w2_s[i] = to_float<T>(reinterpret_cast<const T*>(a.w2)[(size_t)(ch0 + c) * R + m]);
  }
  if (KL * NPT != N)  // the lanes' slices reach past the head's channels: those places stay zero for the whole pass
    for (int i = tid; i < 2 * BUF; i += blockDim.x) sm[i] = 0.f;
  grid_dependency_wait();
  const int row0 = a.cu_q[seq], T_len = a.seq_qlen[seq], slot = a.seq_slot[seq];
  const int n_chunks = (T_len + TC - 1) / TC;
  const bool consumer = tid < cons;
  float* st = a.state + (((size_t)slot * a.H + head) * N) * N;

  // consumer: value channels col0 .. col0 + CPT - 1, key channels key0 .. key0 + NPT - 1
  const int col0 = (tid / KL) * CPT, slice = tid % KL;
  const int key0 = slice * NPT;
  bool on[CPT];
  float S[CPT][NPT];
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2) {
    on[c2] = consumer && col0 + c2 < N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[c2][i] = (on[c2] && key0 + i < N) ? st[(size_t)(key0 + i) * N + col0 + c2] : 0.f;
  }

  // producer
  const int pt = tid - cons, plane = pt & 31, pwarp = pt >> 5;
  const T* rp = reinterpret_cast<const T*>(a.r);
  const T* kp = reinterpret_cast<const T*>(a.k);
  const T* vp = reinterpret_cast<const T*>(a.v);
  const T* gp = reinterpret_cast<const T*>(a.g);
  const T* ap = reinterpret_cast<const T*>(a.rate);
  const T* lp = reinterpret_cast<const T*>(a.lora);
  T* outp = reinterpret_cast<T*>(a.out);
  __syncthreads();

  for (int c = 0; c < n_chunks + 2; ++c) {
    if (consumer) {
      const int cc = c - 1;  // the chunk to scan
      if (cc >= 0 && cc < n_chunks) {
        const int nt = min(TC, T_len - cc * TC);
        const float* buf = sm + (cc & 1) * BUF;
        const float* v_s = buf + 5 * TC * VS;
        float* o_c = o_s + (cc & 1) * TC * N;
        for (int t = 0; t < nt; ++t) {
          const int at = t * VS + slice * SL;
          const float4* r4 = reinterpret_cast<const float4*>(buf + at);
          const float4* k4 = reinterpret_cast<const float4*>(buf + TC * VS + at);
          const float4* w4 = reinterpret_cast<const float4*>(buf + 2 * TC * VS + at);
          const float4* u4 = reinterpret_cast<const float4*>(buf + 3 * TC * VS + at);
          float vj[CPT], o[CPT];
#pragma unroll
          for (int c2 = 0; c2 < CPT; ++c2) vj[c2] = on[c2] ? v_s[t * N + col0 + c2] : 0.f;
          scan_token<RULE, NPT, CPT>(S, r4, k4, w4, u4, reinterpret_cast<const float4*>(buf + 4 * TC * VS + at), vj, KL, o);
#pragma unroll
          for (int c2 = 0; c2 < CPT; ++c2)
            if (on[c2] && slice == 0) o_c[t * N + col0 + c2] = o[c2];
        }
      }
    } else {
      // -- finish chunk c - 2: per head divide by the root mean square, weight, gate, scale ----------
      const int fc = c - 2;
      if (fc >= 0 && fc < n_chunks) {
        const int nt = min(TC, T_len - fc * TC), t0 = fc * TC;
        const float* o_c = o_s + (fc & 1) * TC * N;
        float* red = red_s + TC;
        for (int t = pwarp; t < nt; t += PROD / 32) {
          float sq = 0.f;
          for (int ch = plane; ch < N; ch += 32) sq += o_c[t * N + ch] * o_c[t * N + ch];
          sq = warp_sum(sq);
          if (plane == 0) red[t] = rsqrtf(sq / (float)N + a.eps);
        }
        producers_sync();
        if (a.vec) {  // four channels at a time, four such pieces requested before the first is used
          const int N4 = N / 4, items = nt * N4;
          for (int i0 = pt; i0 < items; i0 += 4 * PROD) {
            float g[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i = i0 + u * PROD;
              if (i < items) load4_el<T>(gp + (size_t)(row0 + t0 + i / N4) * a.g_stride + ch0 + 4 * (i % N4), g[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i = i0 + u * PROD;
              if (i >= items) continue;
              const int t = i / N4, ch = 4 * (i % N4);
              float o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float gate = RULE == 1 ? sigmoidf(g[u][e]) : g[u][e] * sigmoidf(g[u][e]);
                o[e] = o_c[t * N + ch + e] * red[t] * a.norm_w[ch0 + ch + e] * gate * a.out_scale;
              }
              store4_el<T>(outp + (size_t)(row0 + t0 + t) * a.out_stride + a.out_col + ch0 + ch, o);
            }
          }
        } else
        for (int i = pt; i < nt * N; i += PROD) {
          const int t = i / N, ch = i % N;
          const size_t row = (size_t)(row0 + t0 + t);
          const float g = to_float<T>(gp[row * a.g_stride + ch0 + ch]);
          const float gate = RULE == 1 ? sigmoidf(g) : g * sigmoidf(g);
          outp[row * a.out_stride + a.out_col + ch0 + ch] =
              from_float<T>(o_c[i] * red[t] * a.norm_w[ch0 + ch] * gate * a.out_scale);
        }
      }
      // -- prepare chunk c ---------------------------------------------------------------------------
      if (c < n_chunks) {
        const int nt = min(TC, T_len - c * TC), t0 = c * TC;
        float* buf = sm + (c & 1) * BUF;
        float* r_s = buf;
        float* k_s = buf + TC * VS;
        float* w_s = buf + 2 * TC * VS;
        float* u_s = buf + 3 * TC * VS;
        float* au_s = buf + 4 * TC * VS;
        float* v_s = buf + 5 * TC * VS;
        producers_sync();  // th_s and red_s of the chunk before are no longer read
        if (a.vec) {  // four channels at a time; two such pieces of every input requested before the first is used
          const int N4 = N / 4, items = nt * N4;
          for (int i0 = pt; i0 < items; i0 += 2 * PROD) {
            float rv[2][4], kv[2][4], vv[2][4], av[2][4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = i0 + u * PROD;
              if (i >= items) continue;
              const size_t row = (size_t)(row0 + t0 + i / N4);
              const int ch = ch0 + 4 * (i % N4);
              load4_el<T>(rp + row * a.r_stride + ch, rv[u]);
              load4_el<T>(kp + row * a.k_stride + ch, kv[u]);
              load4_el<T>(vp + row * a.v_stride + ch, vv[u]);
              if (RULE == 1) load4_el<T>(ap + row * a.rate_stride + ch, av[u]);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = i0 + u * PROD;
              if (i >= items) continue;
              const int t = i / N4, ch = 4 * (i % N4);
              const int at = t * VS + (ch / NPT) * SL + (ch % NPT);
              *reinterpret_cast<float4*>(r_s + at) = make_float4(rv[u][0], rv[u][1], rv[u][2], rv[u][3]);
              *reinterpret_cast<float4*>(k_s + at) = make_float4(kv[u][0], kv[u][1], kv[u][2], kv[u][3]);
              *reinterpret_cast<float4*>(v_s + t * N + ch) = make_float4(vv[u][0], vv[u][1], vv[u][2], vv[u][3]);
              if (RULE == 1) *reinterpret_cast<float4*>(au_s + at) = make_float4(av[u][0], av[u][1], av[u][2], av[u][3]);
            }
          }
        } else
        for (int i = pt; i < nt * N; i += PROD) {
          const int t = i / N, ch = i % N;
          const size_t row = (size_t)(row0 + t0 + t);
          const int at = t * VS + (ch / NPT) * SL + (ch % NPT);
          r_s[at] = to_float<T>(rp[row * a.r_stride + ch0 + ch]);
          k_s[at] = to_float<T>(kp[row * a.k_stride + ch0 + ch]);
          v_s[i] = to_float<T>(vp[row * a.v_stride + ch0 + ch]);
          if (RULE == 1) au_s[at] = to_float<T>(ap[row * a.rate_stride + ch0 + ch]);  // the raw rate, for now
        }
        for (int i = pt; i < nt * R; i += PROD) {
          const int t = i / R, m = i % R;
          th_s[i] = round_to<T>(tanhf(to_float<T>(lp[(size_t)(row0 + t0 + t) * a.lora_stride + m])));
        }
        producers_sync();
        if (RULE == 1) {  // per token: sum of squared key channels
          for (int t = pwarp; t < nt; t += PROD / 32) {
            float sq = 0.f;
            for (int ch = plane; ch < N; ch += 32) {
              const float kv = k_s[t * VS + (ch / NPT) * SL + (ch % NPT)];
              sq += kv * kv;
            }
            sq = warp_sum(sq);
            if (plane == 0) red_s[t] = rsqrtf(sq + 1e-6f);
          }
          producers_sync();
        }
        for (int i = pt; i < nt * N; i += PROD) {
          const int t = i / N, ch = i % N;
          const int at = t * VS + (ch / NPT) * SL + (ch % NPT);
          float z = 0.f;
          for (int m = 0; m < R; ++m) z += th_s[t * R + m] * w2_s[m * N + ch];
          z += a.w0[ch0 + ch];
          if (RULE == 1) {
            w_s[at] = expf(-a.decay_scale * sigmoidf(z));
            const float u = k_s[at] * red_s[t];
            u_s[at] = u;
            au_s[at] = sigmoidf(au_s[at] + a.rate_bias[ch0 + ch]) * u;
          } else {
            w_s[at] = expf(-expf(z));
            u_s[at] = a.bonus[ch0 + ch] * k_s[at];
          }
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2)
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      if (on[c2] && key0 + i < N) st[(size_t)(key0 + i) * N + col0 + c2] = S[c2][i];
  if (a.last_rows && head == 0 && T_len > 0) {
    const T* last = reinterpret_cast<const T*>(a.last_rows) + (size_t)(row0 + T_len - 1) * a.last_stride;
    float* dst = a.last_state + (size_t)slot * a.C;
    for (int ch = tid; ch < a.C; ch += blockDim.x) dst[ch] = to_float<T>(last[ch]);
  }
}

template <typename T, int RULE, int NPT, int CPT, int TC, int PROD, int MAXT>
int launch_recurrence(const ScanArgs& a, cudaStream_t stream) {
  int KL = 1;
  while (KL * NPT < a.N) KL <<= 1;
  const int cons = (((a.N + CPT - 1) / CPT * KL + 31) / 32) * 32;
  if (cons + PROD > MAXT) return -2;
  const size_t buf = (size_t)5 * TC * KL * (NPT + 4) + (size_t)TC * a.N;
  const size_t smem = (2 * buf + (size_t)2 * TC * a.N + (size_t)a.R * a.N + (size_t)TC * a.R + 2 * TC) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  auto kern = recurrence_kernel<T, RULE, NPT, CPT, TC, PROD, MAXT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(a.n_seqs * a.H), dim3(cons + PROD), smem, stream, a, KL, cons);
}

template <typename T, int RULE>
int pick_recurrence(const ScanArgs& a, cudaStream_t stream) {
  if (a.N <= 64) return launch_recurrence<T, RULE, 16, 2, 32, 256, 384>(a, stream);
  if (a.N <= 128) return launch_recurrence<T, RULE, 32, 2, 16, 128, 384>(a, stream);
  // larger heads: four columns a thread; the state then spills from the registers, which is slow and right
  if (a.N <= 256) return launch_recurrence<T, RULE, 32, 4, 8, 128, 640>(a, stream);
  return -2;  // a head's state no longer fits one block
}

// ---------------------------------------------------------------------------------------------------
// An option for steps of many tokens per sequence (off by default: measured on 2,048 tokens of 8 heads of 64
// channels it takes 1.15 ms with chunks of 32 tokens and 1.78 ms with chunks of 16, the fused kernel 1.24 ms
// alone and 5 % less inside a prompt step): the same work as three kernels. What does not depend on the state
// (decays, unit keys, rates; the per-head norm, weight and gate of the outputs) runs over all rows at
// once on every SM; between them the scan kernel only streams the prepared float32 vectors into shared
// memory with cp.async, one chunk ahead, and applies the rule. Every sum is the one the fused kernel
// forms, in the same order, so the two agree to the bit.
//   prep [rows, H, 6, N] float32: r, k, decay, u (or bonus * k), rate * u, v
//   o    [rows, H * N]  float32: the raw outputs
// ---------------------------------------------------------------------------------------------------
template <typename T, int RULE>
__global__ void recurrence_prepare_kernel(ScanArgs a, float* __restrict__ prep) {
  extern __shared__ float sp[];  // [R] tanh of the low-rank input, then one float
  grid_launch_dependents();
  grid_dependency_wait();
  const int N = a.N, R = a.R;
  const size_t row = blockIdx.x;
  const int head = blockIdx.y, ch0 = head * N;
  const int tid = threadIdx.x, lane = tid & 31;
  const T* lp = reinterpret_cast<const T*>(a.lora);
  for (int m = tid; m < R; m += blockDim.x) sp[m] = round_to<T>(tanhf(to_float<T>(lp[row * a.lora_stride + m])));
  const T* kp = reinterpret_cast<const T*>(a.k) + row * a.k_stride + ch0;
  if (RULE == 1 && tid < 32) {
    float sq = 0.f;
    for (int c = lane; c < N; c += 32) {
      const float kv = to_float<T>(kp[c]);
      sq += kv * kv;
    }
    sq = warp_sum(sq);
    if (lane == 0) sp[R] = rsqrtf(sq + 1e-6f);
  }
  __syncthreads();
  float* dst = prep + (row * a.H + head) * 6 * N;
  const T* w2 = reinterpret_cast<const T*>(a.w2);
  for (int c = tid; c < N; c += blockDim.x) {
    const float kv = to_float<T>(kp[c]);
    float z = 0.f;
    for (int m = 0; m < R; ++m) z += sp[m] * to_float<T>(w2[(size_t)(ch0 + c) * R + m]);
    z += a.w0[ch0 + c];
    dst[c] = to_float<T>(reinterpret_cast<const T*>(a.r)[row * a.r_stride + ch0 + c]);
    dst[N + c] = kv;
    dst[5 * N + c] = to_float<T>(reinterpret_cast<const T*>(a.v)[row * a.v_stride + ch0 + c]);
    if (RULE == 1) {
      dst[2 * N + c] = expf(-a.decay_scale * sigmoidf(z));
      const float u = kv * sp[R];
      dst[3 * N + c] = u;
      dst[4 * N + c] =
          sigmoidf(to_float<T>(reinterpret_cast<const T*>(a.rate)[row * a.rate_stride + ch0 + c]) + a.rate_bias[ch0 + c]) * u;
    } else {
      dst[2 * N + c] = expf(-expf(z));
      dst[3 * N + c] = a.bonus[ch0 + c] * kv;
      dst[4 * N + c] = 0.f;
    }
  }
}

template <typename T, int RULE, int NPT, int CPT, int TC, int MAXT>
__global__ void __launch_bounds__(MAXT)
recurrence_scan_kernel(ScanArgs a, const float* __restrict__ prep, float* __restrict__ o_out, int KL) {
  constexpr int SL = NPT + 4;
  extern __shared__ __align__(16) float sm[];
  const int N = a.N;
  const int VS = KL * SL;
  const int BUF = 5 * TC * VS + TC * N;
  grid_launch_dependents();
  const int seq = blockIdx.x / a.H, head = blockIdx.x % a.H;
  const int tid = threadIdx.x;
  if (KL * NPT != N)
    for (int i = tid; i < 2 * BUF; i += blockDim.x) sm[i] = 0.f;
  grid_dependency_wait();
  const int row0 = a.cu_q[seq], T_len = a.seq_qlen[seq], slot = a.seq_slot[seq];
  const int n_chunks = (T_len + TC - 1) / TC;
  float* st = a.state + (((size_t)slot * a.H + head) * N) * N;
  const int col0 = (tid / KL) * CPT, slice = tid % KL;
  const int key0 = slice * NPT;
  bool on[CPT];
  float S[CPT][NPT];
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2) {
    on[c2] = col0 + c2 < N;
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[c2][i] = (on[c2] && key0 + i < N) ? st[(size_t)(key0 + i) * N + col0 + c2] : 0.f;
  }
  __syncthreads();
  const int N4 = N / 4;
  auto issue = [&](int c) {  // chunk c -> buffer c & 1, 16 bytes a request
    const int nt = min(TC, T_len - c * TC);
    float* buf = sm + (c & 1) * BUF;
    for (int i = tid; i < nt * 6 * N4; i += blockDim.x) {
      const int t = i / (6 * N4), rem = i % (6 * N4), vec = rem / N4, ch = 4 * (rem % N4);
      const float* src = prep + (((size_t)(row0 + c * TC + t)) * a.H + head) * 6 * N + vec * N + ch;
      float* dst = vec < 5 ? buf + vec * TC * VS + t * VS + (ch / NPT) * SL + (ch % NPT) : buf + 5 * TC * VS + t * N + ch;
      cp_async_16(dst, src);
    }
    cp_async_commit();
  };
  if (n_chunks > 0) issue(0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) {
      issue(c + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int nt = min(TC, T_len - c * TC);
    const float* buf = sm + (c & 1) * BUF;
    const float* v_s = buf + 5 * TC * VS;
    for (int t = 0; t < nt; ++t) {
      const int at = t * VS + slice * SL;
      float vj[CPT], o[CPT];
#pragma unroll
      for (int c2 = 0; c2 < CPT; ++c2) vj[c2] = on[c2] ? v_s[t * N + col0 + c2] : 0.f;
      scan_token<RULE, NPT, CPT>(S, reinterpret_cast<const float4*>(buf + at), reinterpret_cast<const float4*>(buf + TC * VS + at),
                            reinterpret_cast<const float4*>(buf + 2 * TC * VS + at),
                            reinterpret_cast<const float4*>(buf + 3 * TC * VS + at),
                            reinterpret_cast<const float4*>(buf + 4 * TC * VS + at), vj, KL, o);
      float* orow = o_out + (size_t)(row0 + c * TC + t) * a.H * N + head * N;
#pragma unroll
      for (int c2 = 0; c2 < CPT; ++c2)
        if (on[c2] && slice == 0) orow[col0 + c2] = o[c2];
    }
    __syncthreads();  // the buffer is free for the chunk after next
  }
#pragma unroll
  for (int c2 = 0; c2 < CPT; ++c2)
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      if (on[c2] && key0 + i < N) st[(size_t)(key0 + i) * N + col0 + c2] = S[c2][i];
  if (a.last_rows && head == 0 && T_len > 0) {
    const T* last = reinterpret_cast<const T*>(a.last_rows) + (size_t)(row0 + T_len - 1) * a.last_stride;
    float* dst = a.last_state + (size_t)slot * a.C;
    for (int ch = tid; ch < a.C; ch += blockDim.x) dst[ch] = to_float<T>(last[ch]);
  }
}

// out = o / sqrt(mean_head(o^2) + eps) * norm_w * gate(g) * out_scale: one warp per (row, head).
template <typename T, int RULE>
__global__ void recurrence_finish_kernel(ScanArgs a, const float* __restrict__ o_in, int rows) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int N = a.N, lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)rows * a.H) return;
  const size_t row = (size_t)(w / a.H);
  const int head = (int)(w % a.H), ch0 = head * N;
  const float* o = o_in + row * a.H * N + ch0;
  float sq = 0.f;
  for (int c = lane; c < N; c += 32) sq += o[c] * o[c];
  sq = warp_sum(sq);
  const float rstd = rsqrtf(sq / (float)N + a.eps);
  const T* gp = reinterpret_cast<const T*>(a.g) + row * a.g_stride + ch0;
  T* outp = reinterpret_cast<T*>(a.out) + row * a.out_stride + a.out_col + ch0;
  for (int c = lane; c < N; c += 32) {
    const float g = to_float<T>(gp[c]);
    const float gate = RULE == 1 ? sigmoidf(g) : g * sigmoidf(g);
    outp[c] = from_float<T>(o[c] * rstd * a.norm_w[ch0 + c] * gate * a.out_scale);
  }
}

template <typename T, int RULE, int NPT, int CPT, int TC, int MAXT>
int launch_split(const ScanArgs& a, float* prep, float* o_scratch, int rows, cudaStream_t stream) {
  int KL = 1;
  while (KL * NPT < a.N) KL <<= 1;
  const int cons = (((a.N + CPT - 1) / CPT * KL + 31) / 32) * 32;
  if (cons > MAXT) return -2;
  const size_t smem = (size_t)2 * (5 * TC * KL * (NPT + 4) + TC * a.N) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  cudaError_t e = launch_pdl(recurrence_prepare_kernel<T, RULE>, dim3(rows, a.H), dim3(a.N <= 32 ? 32 : 64),
                             (size_t)(a.R + 1) * sizeof(float), stream, a, prep);
  if (e != cudaSuccess) return (int)e;
  auto kern = recurrence_scan_kernel<T, RULE, NPT, CPT, TC, MAXT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  e = launch_pdl(kern, dim3(a.n_seqs * a.H), dim3(cons), smem, stream, a, (const float*)prep, o_scratch, KL);
  if (e != cudaSuccess) return (int)e;
  const long long warps = (long long)rows * a.H;
  return (int)launch_pdl(recurrence_finish_kernel<T, RULE>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, a,
                         (const float*)o_scratch, rows);
}

template <typename T, int RULE>
int pick_split(const ScanArgs& a, float* prep, float* o_scratch, int rows, cudaStream_t stream) {
  if (a.N <= 64) return launch_split<T, RULE, 16, 2, 32, 128>(a, prep, o_scratch, rows, stream);
  if (a.N <= 128) return launch_split<T, RULE, 32, 2, 16, 256>(a, prep, o_scratch, rows, stream);
  return -2;
}

}  // namespace

KRK_API int krk_token_shift(void* out, const void* h, int h_stride, float* last_state, const float* mu, int n_mix,
                            int C, int rows, const int* row_seq, const int* cu_q, const int* seq_slot, int dtype,
                            cudaStream_t stream, int store) {
  if (rows == 0) return 0;
  const int threads = C >= 1024 ? 256 : 128;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(token_shift_kernel<float>, dim3(rows), dim3(threads), 0, stream, (float*)out, (const float*)h,
                           h_stride, last_state, mu, n_mix, C, rows, row_seq, cu_q, seq_slot, store);
  return (int)launch_pdl(token_shift_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, (bf16*)out, (const bf16*)h,
                         h_stride, last_state, mu, n_mix, C, rows, row_seq, cu_q, seq_slot, store);
}

KRK_API int krk_linear_recurrence(int rule, const void* r, int r_stride, const void* k, int k_stride, const void* v,
                                  int v_stride, const void* g, int g_stride, const void* rate, int rate_stride,
                                  const void* lora, int lora_stride, const void* w2, const float* w0,
                                  const float* rate_bias, const float* bonus, const float* norm_w, float* state,
                                  const void* last_rows, int last_stride, int C, float* last_state, void* out,
                                  int out_stride, int out_col, float out_scale, float eps, float decay_scale, int H, int N,
                                  int R, int n_seqs, const int* cu_q, const int* seq_qlen, const int* seq_slot, int rows,
                                  float* prep, float* o_scratch, int dtype, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  ScanArgs a;
  a.r = r; a.k = k; a.v = v; a.g = g; a.rate = rate; a.lora = lora;
  a.r_stride = r_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.g_stride = g_stride;
  a.rate_stride = rate_stride; a.lora_stride = lora_stride;
  a.w2 = w2; a.w0 = w0; a.rate_bias = rate_bias; a.bonus = bonus; a.norm_w = norm_w; a.state = state;
  a.last_rows = last_rows; a.last_stride = last_stride; a.C = C; a.last_state = last_state;
  a.out = out; a.out_stride = out_stride; a.out_col = out_col; a.out_scale = out_scale; a.eps = eps;
  a.decay_scale = decay_scale; a.H = H; a.N = N; a.R = R; a.n_seqs = n_seqs;
  a.cu_q = cu_q; a.seq_qlen = seq_qlen; a.seq_slot = seq_slot;
  {
    const uintptr_t mask = dtype == KRK_DTYPE_F32 ? 15 : 7;
    const uintptr_t ptrs = (uintptr_t)r | (uintptr_t)k | (uintptr_t)v | (uintptr_t)g | (uintptr_t)rate | (uintptr_t)out;
    const int strides = r_stride | k_stride | v_stride | g_stride | rate_stride | out_stride | out_col | N;
    a.vec = (ptrs & mask) == 0 && (strides & 3) == 0;
  }
  if (rule != 0 && rule != 1) return -2;
  if (rule == 1 && (!rate || !rate_bias)) return -2;
  if (rule == 0 && !bonus) return -2;
  if (prep && o_scratch && N % 4 == 0 && rows > 0) {
    // steps of many tokens: prepare, scan, finish (scratch of rows * H * 6 * N and rows * H * N floats)
    int rc;
    if (dtype == KRK_DTYPE_F32)
      rc = rule == 1 ? pick_split<float, 1>(a, prep, o_scratch, rows, stream) : pick_split<float, 0>(a, prep, o_scratch, rows, stream);
    else
      rc = rule == 1 ? pick_split<bf16, 1>(a, prep, o_scratch, rows, stream) : pick_split<bf16, 0>(a, prep, o_scratch, rows, stream);
    if (rc != -2) return rc;
  }
  if (dtype == KRK_DTYPE_F32)
    return rule == 1 ? pick_recurrence<float, 1>(a, stream) : pick_recurrence<float, 0>(a, stream);
  return rule == 1 ? pick_recurrence<bf16, 1>(a, stream) : pick_recurrence<bf16, 0>(a, stream);
}
