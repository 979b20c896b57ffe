// Recurrent mixers whose state is a matrix per sequence and head, with gates that depend on the token.
//
//   matrix_memory (mLSTM):  m_t = max(f_t + m_(t-1), i_t)                               (m_0 = 0, S_0 = 0, n_0 = 0)
//                           S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t the same with k_t alone
//                           o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//                           i_t = cap tanh(a_t / cap),  f_t = logsigmoid(cap tanh(b_t / cap))   (a, b: the gate projections)
//   delta_rule:             S <- g_t * S (a decay per key channel, on the rows of S);  u = beta_t (v_t - S^T k_t);
//                           S <- S + k_t u^T;  o_t = S^T q_t                             (the read-out sees the write)
//                           g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias)),  beta_t = sigmoid(b_t)
//   short_conv:             per channel, y_t = silu(sum_j w[c, j] x_(t - taps + 1 + j)) with zeros before the start; the first
//                           channels may be `unit_heads` heads that are then made unit vectors (x / sqrt(sum x^2 + eps)), the
//                           first `scaled_heads` of them times a constant; channels after the convolved ones pass a sigmoid
//   conv_state:             the last taps - 1 inputs of every sequence, kept for the next step
//   head_norm_gate:         out = o / sqrt(mean_head(o^2) + eps) * w * sigmoid(gate)
//
// Everything after the projections is 32-bit: gates, their logarithms and exponentials, the unit vectors, the state,
// the read-out and the per-head norm.  The columns of S (one per value entry) do not depend on one another, so a
// block owns (sequence, head, 16 value columns) and walks the sequence's rows of this step in order; eight lanes
// share a column, each with an eighth of its key entries in registers (four neighbours at a time), and meet by three shuffles for the two dot
// products a row needs.  The rows' q, k and gates are staged 16 (or 8) rows at a time in shared memory, where the
// scalar recurrences (the running maximum) and the transcendental functions are done once per block.  One row is
// the same walk, so decoding, whole prompts and prompts in portions give the same bits.  The state of a slot is
// [heads, dv, dk] (a column's key entries side by side), then for the matrix memory n [heads, tiles, dk] and
// m [heads, tiles] (a copy per block of 16 columns, so that no block reads what another writes).
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int COLS = 16;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

struct RecArgs {
  const void* q; const void* k; const void* v;
  int64_t ld_q, ld_k, ld_v;            // head h reads the query/key head h / group at column (h / group) * dk
  const float* gates; int64_t ld_gates;   // matrix memory: [rows, 2 heads] (input | forget), raw; delta rule: [rows, heads * dk], raw
  const float* beta; int64_t ld_beta;     // delta rule: [rows, heads], already sigmoid
  const void* a_log; const void* dt_bias; int params_f32;
  float* out; int64_t ld_out;          // [rows, heads * dv], raw read-out
  float* state; int64_t state_stride;
  const int* seq_starts; const int* seq_slots;
  int heads, group, dk, dv, tiles;
  int gates_ready;                     // delta rule: `gates` already holds the decays themselves (see decay_gate)
  float q_scale, cap;
};

template <typename TI, int EPL, int MODE>
__global__ void __launch_bounds__(128) recurrence_kernel(const RecArgs p) {
  constexpr int DKP = EPL * 8, TC = EPL >= 64 ? 4 : (EPL >= 32 ? 8 : 16);
  constexpr int PER = TC * DKP / 128;          // staged q (k, gate) entries a thread carries from global to shared memory
  constexpr int VPER = TC * COLS >= 128 ? TC * COLS / 128 : 1;
  __shared__ __align__(16) float sq[TC][DKP], sk[TC][DKP];
  __shared__ __align__(16) float sg[MODE == 1 ? TC : 1][MODE == 1 ? DKP : 4];
  __shared__ float sbias[MODE == 1 ? DKP : 1];
  __shared__ float sv[TC][COLS];
  __shared__ float s_a[TC], s_b[TC], s_c[TC], s_i[TC], s_f[TC];
  __shared__ float s_m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, sub = lane & 7, grp = lane >> 3;
  const int col = blockIdx.x * COLS + warp * 4 + grp;
  const int h = blockIdx.y, s = blockIdx.z, qh = h / p.group;
  const int dk = p.dk, dv = p.dv;
  float decay_rate = 0.f;
  if (MODE == 1) {                             // parameters do not depend on the kernel before
    decay_rate = expf(load_param(p.a_log, h, p.params_f32));
    for (int d = tid; d < DKP; d += 128) sbias[d] = d < dk ? load_param(p.dt_bias, h * dk + d, p.params_f32) : 0.f;
  }
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = p.seq_starts[s], row1 = p.seq_starts[s + 1];
  float* st = p.state + (int64_t)p.seq_slots[s] * p.state_stride;
  const bool col_ok = col < dv;
  float* S_g = st + ((int64_t)h * dv + (col_ok ? col : 0)) * dk;
  float* n_g = st + (int64_t)p.heads * dv * dk + ((int64_t)h * p.tiles + blockIdx.x) * dk;
  float* m_g = st + (int64_t)p.heads * dv * dk + (int64_t)p.heads * p.tiles * dk + (int64_t)h * p.tiles + blockIdx.x;
  // a lane's entries: four neighbouring key entries at a time, so that it reads q, k and the decays as 16-byte pieces
  // and the eight lanes of a column read 128 bytes side by side: entry e of lane `sub` is key entry ((e / 4) * 8 + sub) * 4 + e % 4
  float S[EPL], N[MODE == 0 ? EPL : 1];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = (((e >> 2) * 8 + sub) << 2) + (e & 3);
    S[e] = (col_ok && d < dk) ? S_g[d] : 0.f;
    if (MODE == 0) N[e] = d < dk ? n_g[d] : 0.f;
  }
  if (MODE == 0 && tid == 0) s_m = *m_g;
  const TI* q = reinterpret_cast<const TI*>(p.q);
  const TI* k = reinterpret_cast<const TI*>(p.k);
  const TI* v = reinterpret_cast<const TI*>(p.v);

  // the next rows' inputs are fetched into registers while the rows before them are walked
  // (as they are stored: a conversion here would wait for the load)
  TI rq[PER], rk[PER], rv[VPER];
  float rg[MODE == 1 ? PER : 1], r0 = 0.f, r1 = 0.f;
  const TI zero = from_f32<TI>(0.f);
  auto fetch = [&](int c0) {
    const int nt = min(TC, row1 - c0);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = tid + j * 128, t = i / DKP, d = i - t * DKP;
      const int64_t r = c0 + t;
      const bool ok = t < nt && d < dk;
      rq[j] = ok ? q[r * p.ld_q + qh * dk + d] : zero;
      rk[j] = ok ? k[r * p.ld_k + qh * dk + d] : zero;
      if (MODE == 1) rg[j] = ok ? p.gates[r * p.ld_gates + h * dk + d] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < VPER; ++j) {
      const int i = tid + j * 128, t = i / COLS, c = blockIdx.x * COLS + (i - t * COLS);
      rv[j] = (t < nt && c < dv) ? v[(int64_t)(c0 + t) * p.ld_v + h * dv + c] : zero;      // (t < nt <= TC also where a block has more threads than values)
    }
    if (tid < nt) {
      if (MODE == 1) {
        r0 = p.beta[(int64_t)(c0 + tid) * p.ld_beta + h];
      } else {
        const float* gr = p.gates + (int64_t)(c0 + tid) * p.ld_gates;
        r0 = gr[h];
        r1 = gr[p.heads + h];
      }
    }
  };
  if (row0 < row1) fetch(row0);

  for (int c0 = row0; c0 < row1; c0 += TC) {
    const int nt = min(TC, row1 - c0);
    __syncthreads();                            // the rows before have been walked
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = tid + j * 128, t = i / DKP, d = i - t * DKP;
      sq[t][d] = to_f32(rq[j]) * p.q_scale;
      sk[t][d] = to_f32(rk[j]);
      if (MODE == 1) sg[t][d] = d >= dk ? 1.f : (p.gates_ready ? rg[j] : expf(-decay_rate * softplus_f(rg[j] + sbias[d])));
    }
#pragma unroll
    for (int j = 0; j < VPER; ++j) {
      const int i = tid + j * 128;
      if (i < TC * COLS) sv[i / COLS][i % COLS] = to_f32(rv[j]);
    }
    if (tid < nt) {
      if (MODE == 1) {
        s_a[tid] = r0;
      } else {                                  // the caps and the logarithm of the forget gate, a thread per row
        s_i[tid] = p.cap * tanhf(r0 / p.cap);
        s_f[tid] = -softplus_f(-p.cap * tanhf(r1 / p.cap));
      }
    }
    __syncthreads();
    if (c0 + TC < row1) fetch(c0 + TC);
    if (MODE == 1) {
      for (int t = warp; t < nt; t += 4) {
        float acc = 0.f;
        for (int d = lane; d < DKP; d += 32) acc = fmaf(sk[t][d], sq[t][d], acc);
        acc = warp_sum(acc);
        if (lane == 0) s_b[t] = acc;
      }
    } else {
      if (tid == 0) {                           // the running maximum is the one thing that goes row by row
        float m = s_m;
        for (int t = 0; t < nt; ++t) {
          const float mn = fmaxf(s_f[t] + m, s_i[t]);
          s_a[t] = m;
          s_c[t] = mn;
          m = mn;
        }
        s_m = m;
      }
      __syncthreads();
      if (tid < nt) {
        const float m_before = s_a[tid], mn = s_c[tid];
        s_a[tid] = expf(s_f[tid] + m_before - mn);
        s_b[tid] = expf(s_i[tid] - mn);
        s_c[tid] = expf(-mn);
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float vj = sv[t][warp * 4 + grp];
      const float4* k4 = reinterpret_cast<const float4*>(sk[t]) + sub;
      const float4* q4 = reinterpret_cast<const float4*>(sq[t]) + sub;
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f, o;       // (two partial sums each: half as long a chain)
      if (MODE == 0) {
        const float keep = s_a[t], take = s_b[t];
        const float tv = take * vj;
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          const float4 kk = k4[j * 8], qq = q4[j * 8];
          float* Sj = S + 4 * j;
          float* Nj = N + 4 * j;
          Sj[0] = fmaf(keep, Sj[0], tv * kk.x); Sj[1] = fmaf(keep, Sj[1], tv * kk.y);
          Sj[2] = fmaf(keep, Sj[2], tv * kk.z); Sj[3] = fmaf(keep, Sj[3], tv * kk.w);
          Nj[0] = fmaf(keep, Nj[0], take * kk.x); Nj[1] = fmaf(keep, Nj[1], take * kk.y);
          Nj[2] = fmaf(keep, Nj[2], take * kk.z); Nj[3] = fmaf(keep, Nj[3], take * kk.w);
          a0 = fmaf(Sj[0], qq.x, a0); a1 = fmaf(Sj[1], qq.y, a1); a0 = fmaf(Sj[2], qq.z, a0); a1 = fmaf(Sj[3], qq.w, a1);
          b0 = fmaf(Nj[0], qq.x, b0); b1 = fmaf(Nj[1], qq.y, b1); b0 = fmaf(Nj[2], qq.z, b0); b1 = fmaf(Nj[3], qq.w, b1);
        }
        float a = a0 + a1, b = b0 + b1;
#pragma unroll
        for (int o2 = 4; o2 > 0; o2 >>= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, o2);
          b += __shfl_xor_sync(0xffffffffu, b, o2);
        }
        o = a / (fmaxf(fabsf(b), s_c[t]) + 1e-6f);
      } else {
        const float4* g4 = reinterpret_cast<const float4*>(sg[t]) + sub;
        float4 kept_k[EPL / 4];
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          const float4 gg = g4[j * 8], kk = k4[j * 8], qq = q4[j * 8];
          kept_k[j] = kk;
          float* Sj = S + 4 * j;
          Sj[0] *= gg.x; Sj[1] *= gg.y; Sj[2] *= gg.z; Sj[3] *= gg.w;
          a0 = fmaf(Sj[0], kk.x, a0); a1 = fmaf(Sj[1], kk.y, a1); a0 = fmaf(Sj[2], kk.z, a0); a1 = fmaf(Sj[3], kk.w, a1);
          b0 = fmaf(Sj[0], qq.x, b0); b1 = fmaf(Sj[1], qq.y, b1); b0 = fmaf(Sj[2], qq.z, b0); b1 = fmaf(Sj[3], qq.w, b1);
        }
        float a = a0 + a1, b = b0 + b1;
#pragma unroll
        for (int o2 = 4; o2 > 0; o2 >>= 1) {
          a += __shfl_xor_sync(0xffffffffu, a, o2);
          b += __shfl_xor_sync(0xffffffffu, b, o2);
        }
        const float u = s_a[t] * (vj - a);
#pragma unroll
        for (int j = 0; j < EPL / 4; ++j) {
          float* Sj = S + 4 * j;
          Sj[0] = fmaf(kept_k[j].x, u, Sj[0]); Sj[1] = fmaf(kept_k[j].y, u, Sj[1]);
          Sj[2] = fmaf(kept_k[j].z, u, Sj[2]); Sj[3] = fmaf(kept_k[j].w, u, Sj[3]);
        }
        o = fmaf(u, s_b[t], b);
      }
      if (sub == 0 && col_ok) p.out[(int64_t)(c0 + t) * p.ld_out + h * dv + col] = o;
    }
  }
  if (row1 > row0) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = (((e >> 2) * 8 + sub) << 2) + (e & 3);
      if (col_ok && d < dk) S_g[d] = S[e];
      if (MODE == 0 && warp == 0 && grp == 0 && d < dk) n_g[d] = N[e];
    }
    if (MODE == 0 && tid == 0) *m_g = s_m;
  }
}

// A block per (row, chunk of columns); a chunk holds whole unit heads.  x: this step's projections; inputs before the
// step's first row come from the sequence's kept inputs [taps - 1, channels] (position p0 - taps + 1 + i at row i), inputs
// before position 0 are zero.  Four columns of a thread are on their way at once: with a few rows a step the kernel is a
// chain of trips to memory and nothing else.
template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T* __restrict__ x, int64_t ld_x, const T* __restrict__ taps, float* __restrict__ y, int64_t ld_y,
                  const float* __restrict__ state, int64_t state_stride, int64_t conv_off, const int* __restrict__ row_seq,
                  const int* __restrict__ row_pos, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                  int channels, int n_taps, int n_sigmoid, int unit_heads, int unit_dim, int scaled_heads, float head_scale,
                  float unit_eps, int chunk) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, s = row_seq[r], pos = row_pos[r], first = seq_starts[s];
  const int p0 = pos - (r - first);
  const float* kept = state + (int64_t)seq_slots[s] * state_stride + conv_off;
  float* yr = y + (int64_t)r * ld_y;
  const int lo = blockIdx.y * chunk, hi = min(lo + chunk, channels + n_sigmoid);
  const int conv_hi = min(hi, channels);
#pragma unroll 4
  for (int c = lo + threadIdx.x; c < conv_hi; c += 128) {
    float acc = 0.f;
    for (int j = 0; j < n_taps; ++j) {
      const int pp = pos - (n_taps - 1) + j;
      float xv = 0.f;
      if (pp >= p0) xv = to_f32(x[(int64_t)(first + pp - p0) * ld_x + c]);
      else if (pp >= 0) xv = kept[(int64_t)(pp - p0 + n_taps - 1) * channels + c];
      acc = fmaf(to_f32(taps[(int64_t)c * n_taps + j]), xv, acc);
    }
    yr[c] = silu_f(acc);
  }
  for (int c = max(lo, channels) + threadIdx.x; c < hi; c += 128) yr[c] = sigmoid_f(to_f32(x[(int64_t)r * ld_x + c]));
  if (unit_heads > 0 && lo < unit_heads * unit_dim) {
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hd_hi = min(unit_heads, hi / unit_dim);
    for (int hd = lo / unit_dim + warp; hd < hd_hi; hd += 4) {
      float* hp = yr + (int64_t)hd * unit_dim;
      float sq = 0.f;
      for (int d = lane; d < unit_dim; d += 32) sq = fmaf(hp[d], hp[d], sq);
      sq = warp_sum(sq);
      const float f = (hd < scaled_heads ? head_scale : 1.f) / sqrtf(sq + unit_eps);
      for (int d = lane; d < unit_dim; d += 32) hp[d] *= f;
    }
  }
}

// g = exp(-exp(A_log_h) softplus(a + dt_bias)) in place on [rows, heads * dk]: for prompts, where every block of a head's
// columns would otherwise work the same decays out again.
__global__ void decay_gate_kernel(float* __restrict__ a, int64_t ld, const void* __restrict__ a_log, const void* __restrict__ dt_bias,
                                  int params_f32, int n_rows, int heads, int dk) {
  pdl_launch_dependents();
  pdl_wait();
  const int width = heads * dk;
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width;
    const int c = (int)(i - r * width);
    float* at = a + r * ld + c;
    *at = expf(-expf(load_param(a_log, c / dk, params_f32)) * softplus_f(*at + load_param(dt_bias, c, params_f32)));
  }
}

// A thread per (sequence, channel): the inputs at the sequence's last taps - 1 positions, from this step's rows or,
// where the step brought fewer, from what was kept before.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int64_t ld_x, float* __restrict__ state, int64_t state_stride,
                                  int64_t conv_off, const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                  int n_seqs, int channels, int n_taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n_seqs * channels) return;
  const int s = (int)(i / channels), c = (int)(i - (int64_t)s * channels);
  const int first = seq_starts[s], n_new = seq_starts[s + 1] - first, keep = n_taps - 1;
  float* kept = state + (int64_t)seq_slots[s] * state_stride + conv_off;
  float old[15];
  for (int j = 0; j < keep; ++j) old[j] = kept[(int64_t)j * channels + c];
  for (int j = 0; j < keep; ++j) {
    const int from_new = n_new - keep + j;          // index among this step's rows, if not negative
    kept[(int64_t)j * channels + c] = from_new >= 0 ? to_f32(x[(int64_t)(first + from_new) * ld_x + c]) : old[j + n_new];
  }
}

// A block per row, a warp per head in turn.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ raw, int64_t ld_raw, const T* __restrict__ gate, int64_t ld_gate,
                      const void* __restrict__ w, int w_f32, int w_per_head, T* __restrict__ out, int64_t ld_out, int heads, int dv,
                      float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int hd = warp; hd < heads; hd += 4) {
    const float* o = raw + (int64_t)r * ld_raw + (int64_t)hd * dv;
    float sq = 0.f;
    for (int d = lane; d < dv; d += 32) sq = fmaf(o[d], o[d], sq);
    sq = warp_sum(sq);
    const float inv = 1.0f / sqrtf(sq / (float)dv + eps);
    for (int d = lane; d < dv; d += 32) {
      float val = o[d] * inv;
      if (w != nullptr) val *= load_param(w, (w_per_head ? hd * dv : 0) + d, w_f32);
      if (gate != nullptr) val *= sigmoid_f(to_f32(gate[(int64_t)r * ld_gate + hd * dv + d]));
      out[(int64_t)r * ld_out + hd * dv + d] = from_f32<T>(val);
    }
  }
}

template <typename TI, int MODE>
int launch_recurrence(const RecArgs& a, int n_seqs, cudaStream_t stream) {
  dim3 grid(a.tiles, a.heads, n_seqs), block(128);
  const int epl = (a.dk + 7) / 8;
  if (epl <= 4) kvad_launch(recurrence_kernel<TI, 4, MODE>, grid, block, 0, stream, a);
  else if (epl <= 8) kvad_launch(recurrence_kernel<TI, 8, MODE>, grid, block, 0, stream, a);
  else if (epl <= 16) kvad_launch(recurrence_kernel<TI, 16, MODE>, grid, block, 0, stream, a);
  else if (epl <= 32) kvad_launch(recurrence_kernel<TI, 32, MODE>, grid, block, 0, stream, a);
  else kvad_launch(recurrence_kernel<TI, 64, MODE>, grid, block, 0, stream, a);
  return 0;
}

}  // namespace

// mode 0: matrix memory, mode 1: delta rule.  in_dtype: the element type of q, k and v.
KVAD_EXPORT int kvad_gated_recurrence(int mode, int in_dtype, const void* q, int64_t ld_q, const void* k, int64_t ld_k, const void* v,
                                      int64_t ld_v, const float* gates, int64_t ld_gates, const float* beta, int64_t ld_beta,
                                      const void* a_log, const void* dt_bias, int params_f32, float* out, int64_t ld_out, float* state,
                                      int64_t state_stride, const int* seq_starts, const int* seq_slots, int n_seqs, int heads,
                                      int kv_heads, int dk, int dv, float q_scale, float cap, int gates_ready, cudaStream_t stream) {
  KVAD_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0 && n_seqs >= 0,
               "gated_recurrence: bad sizes heads=%d kv_heads=%d dk=%d dv=%d", heads, kv_heads, dk, dv);
  KVAD_REQUIRE(dk <= 512, "gated_recurrence: heads of up to 512 key entries, not %d", dk);
  KVAD_REQUIRE(mode == 0 || mode == 1, "gated_recurrence: mode %d", mode);
  KVAD_REQUIRE(q && k && v && gates && out && state && seq_starts && seq_slots, "gated_recurrence: a pointer is missing");
  KVAD_REQUIRE(mode == 0 || (beta && a_log && dt_bias), "gated_recurrence: the delta rule needs beta, A_log and dt_bias");
  KVAD_REQUIRE(mode == 1 || cap > 0.f, "gated_recurrence: the gate cap must be positive");
  if (n_seqs == 0) return KVAD_OK;
  RecArgs a;
  a.q = q; a.k = k; a.v = v; a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v;
  a.gates = gates; a.ld_gates = ld_gates; a.beta = beta; a.ld_beta = ld_beta;
  a.a_log = a_log; a.dt_bias = dt_bias; a.params_f32 = params_f32;
  a.out = out; a.ld_out = ld_out; a.state = state; a.state_stride = state_stride;
  a.seq_starts = seq_starts; a.seq_slots = seq_slots;
  a.heads = heads; a.group = heads / kv_heads; a.dk = dk; a.dv = dv; a.tiles = (dv + COLS - 1) / COLS;
  a.q_scale = q_scale; a.cap = cap; a.gates_ready = gates_ready;
  if (in_dtype == KVAD_DTYPE_F32) {
    if (mode == 0) launch_recurrence<float, 0>(a, n_seqs, stream); else launch_recurrence<float, 1>(a, n_seqs, stream);
  } else if (in_dtype == KVAD_DTYPE_BF16) {
    if (mode == 0) launch_recurrence<__nv_bfloat16, 0>(a, n_seqs, stream); else launch_recurrence<__nv_bfloat16, 1>(a, n_seqs, stream);
  } else {
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "gated_recurrence: unknown dtype %d", in_dtype);
  }
  KVAD_CHECK_LAUNCH("gated_recurrence");
  return KVAD_OK;
}

// floats a slot's state takes: mode 0 the matrices, n and m per block of columns; mode 1 the matrices.
KVAD_EXPORT int kvad_gated_recurrence_state(int mode, int heads, int dk, int dv) {
  const int tiles = (dv + COLS - 1) / COLS;
  return heads * dv * dk + (mode == 0 ? heads * tiles * (dk + 1) : 0);
}

KVAD_EXPORT int kvad_decay_gate(float* a, int64_t ld, const void* a_log, const void* dt_bias, int params_f32, int n_rows, int heads, int dk,
                                cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && heads > 0 && dk > 0 && a && a_log && dt_bias && ld >= (int64_t)heads * dk, "decay_gate: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * heads * dk;
  const int64_t blocks = (total + 255) / 256;
  kvad_launch(decay_gate_kernel, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(256), 0, stream, a, ld, a_log, dt_bias, params_f32,
              n_rows, heads, dk);
  KVAD_CHECK_LAUNCH("decay_gate");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_short_conv(int dtype, const void* x, int64_t ld_x, const void* taps, float* y, int64_t ld_y, const float* state,
                                int64_t state_stride, int64_t conv_off, const int* row_seq, const int* row_pos, const int* seq_starts,
                                const int* seq_slots, int n_rows, int channels, int n_taps, int n_sigmoid, int unit_heads, int unit_dim,
                                int scaled_heads, float head_scale, float unit_eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && channels > 0 && n_taps >= 1 && n_taps <= 16 && n_sigmoid >= 0, "short_conv: bad sizes");
  KVAD_REQUIRE(unit_heads >= 0 && (int64_t)unit_heads * unit_dim <= channels && scaled_heads <= unit_heads, "short_conv: the unit heads do not fit the channels");
  if (n_rows == 0) return KVAD_OK;
  // columns in chunks of at least 512 that hold whole unit heads (one chunk where the heads do not allow it)
  const int total = channels + n_sigmoid;
  int chunk = total;
  if (unit_heads == 0) chunk = 512;
  else if (unit_dim <= 4096) chunk = (512 + unit_dim - 1) / unit_dim * unit_dim;
  dim3 grid(n_rows, (total + chunk - 1) / chunk), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(short_conv_kernel<float>, grid, block, 0, stream, (const float*)x, ld_x, (const float*)taps, y, ld_y, state, state_stride,
                conv_off, row_seq, row_pos, seq_starts, seq_slots, channels, n_taps, n_sigmoid, unit_heads, unit_dim, scaled_heads, head_scale, unit_eps, chunk);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(short_conv_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ld_x, (const __nv_bfloat16*)taps, y, ld_y,
                state, state_stride, conv_off, row_seq, row_pos, seq_starts, seq_slots, channels, n_taps, n_sigmoid, unit_heads, unit_dim,
                scaled_heads, head_scale, unit_eps, chunk);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "short_conv: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("short_conv");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_conv_state(int dtype, const void* x, int64_t ld_x, float* state, int64_t state_stride, int64_t conv_off,
                                const int* seq_starts, const int* seq_slots, int n_seqs, int channels, int n_taps, cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && channels > 0 && n_taps >= 1 && n_taps <= 16, "conv_state: bad sizes");
  if (n_seqs == 0 || n_taps == 1) return KVAD_OK;
  const int64_t total = (int64_t)n_seqs * channels;
  dim3 grid((unsigned)((total + 127) / 128)), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(conv_state_kernel<float>, grid, block, 0, stream, (const float*)x, ld_x, state, state_stride, conv_off, seq_starts, seq_slots,
                n_seqs, channels, n_taps);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(conv_state_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ld_x, state, state_stride, conv_off,
                seq_starts, seq_slots, n_seqs, channels, n_taps);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "conv_state: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("conv_state");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_head_norm_gate(int dtype, const float* raw, int64_t ld_raw, const void* gate, int64_t ld_gate, const void* w, int w_f32,
                                    int w_per_head, void* out, int64_t ld_out, int n_rows, int heads, int dv, float eps,
                                    cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && heads > 0 && dv > 0 && raw && out, "head_norm_gate: bad arguments");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, raw, ld_raw, (const float*)gate, ld_gate, w, w_f32, w_per_head,
                (float*)out, ld_out, heads, dv, eps);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, raw, ld_raw, (const __nv_bfloat16*)gate, ld_gate, w, w_f32,
                w_per_head, (__nv_bfloat16*)out, ld_out, heads, dv, eps);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "head_norm_gate: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("head_norm_gate");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
