// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        (S: [dk, dv] per sequence and head, 32-bit, kept in the cache)
//   o_t = S_t^T q_t
//
// with q and k turned by the row's position first (rotary, pairs half apart or interleaved, over the first
// `rot_dims` entries; angles, sines and the turned values in 32-bit), k scaled by `k_scale` after turning,
// and the output optionally divided by its root mean square per head and multiplied by silu(gate) where it
// is written.  Everything after the projections runs in 32-bit.
//
// A block owns one (sequence, head) and walks the sequence's rows of this step in order, 16 at a time: the
// block turns and stages the 16 rows' q, k, v in shared memory, then every thread carries its share of the
// state through them - thread (v, s) holds S[s * DPT .. s * DPT + DPT - 1][v] in registers, the `split`
// threads of a column are neighbouring lanes and meet by shuffles - and the 16 outputs are normalised,
// gated and written.  A single-token row is the same walk with one row, so decoding and prompts (whole or
// in portions) give the same bits.  The state is read from the sequence's slot at the start and written back
// at the end.
#include "common.cuh"

using namespace kvad;

namespace {

constexpr int TB = 16;

struct RetentionArgs {
  const void* q; const void* k; const void* v; const void* gate;
  int64_t ld_q, ld_k, ld_v, ld_gate;
  void* out; int64_t ld_out;
  float* state;                         // [slots, heads, dk, dv]
  const int* seq_starts; const int* kv_lens; const int* seq_slots;
  const float* decay;                   // [heads]
  const float* inv_freq;                // [rot_dims / 2] or null
  int rot_dims, interleaved;
  int heads, dk, dv, split;
  float k_scale, eps;
  int unit_norm;
};

// (the more state a thread holds, the fewer threads a block may have: registers)
constexpr int max_threads(int dpt) { return dpt == 16 ? 1024 : (dpt <= 32 ? 512 : 256); }

template <typename T, int DPT>
__global__ void __launch_bounds__(max_threads(DPT)) retention_kernel(const RetentionArgs a) {
  extern __shared__ float smem[];
  const int dk = a.dk, dv = a.dv, split = a.split, dkp = split * DPT;
  float* qs = smem;                     // [TB][dkp]
  float* ks = qs + TB * dkp;            // [TB][dkp]
  float* vs = ks + TB * dkp;            // [TB][dv]
  float* os = vs + TB * dv;             // [TB][dv]
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthreads = blockDim.x;
  const int start = a.seq_starts[s], n_new = a.seq_starts[s + 1] - start;
  const int pos0 = a.kv_lens[s] - n_new;
  const int vi = tid / split, si = tid - vi * split;
  const bool owner = vi < dv;
  float* st = a.state + ((int64_t)a.seq_slots[s] * a.heads + h) * dk * dv;
  const float decay = a.decay[h];
  float S[DPT];
#pragma unroll
  for (int j = 0; j < DPT; ++j) {
    const int d = si * DPT + j;
    S[j] = (owner && d < dk) ? st[(int64_t)d * dv + vi] : 0.f;
  }
  const T* q = (const T*)a.q;
  const T* k = (const T*)a.k;
  const T* v = (const T*)a.v;
  const T* gate = (const T*)a.gate;
  T* out = (T*)a.out;
  const int half = a.rot_dims / 2;
  for (int t0 = 0; t0 < n_new; t0 += TB) {
    const int nb = n_new - t0 < TB ? n_new - t0 : TB;
    __syncthreads();                                            // the rows before have been used up
    for (int i = tid; i < nb * dkp; i += nthreads) {
      const int t = i / dkp, d = i - t * dkp;
      float qv = 0.f, kv = 0.f;
      if (d < dk) {
        const int64_t row = start + t0 + t;
        const T* qr = q + row * a.ld_q + (int64_t)h * dk;
        const T* kr = k + row * a.ld_k + (int64_t)h * dk;
        qv = to_f32(qr[d]);
        kv = to_f32(kr[d]);
        if (a.inv_freq != nullptr && d < a.rot_dims) {
          int p, other;
          bool first;
          if (a.interleaved) { p = d >> 1; first = (d & 1) == 0; other = d ^ 1; }
          else { first = d < half; p = first ? d : d - half; other = first ? d + half : d - half; }
          float sn, cs;
          sincosf((float)(pos0 + t0 + t) * a.inv_freq[p], &sn, &cs);
          const float qo = to_f32(qr[other]), ko = to_f32(kr[other]);
          qv = first ? qv * cs - qo * sn : qv * cs + qo * sn;
          kv = first ? kv * cs - ko * sn : kv * cs + ko * sn;
        }
        kv *= a.k_scale;
      }
      qs[i] = qv;
      ks[i] = kv;
    }
    for (int i = tid; i < nb * dv; i += nthreads) {
      const int t = i / dv, d = i - t * dv;
      vs[i] = to_f32(v[(int64_t)(start + t0 + t) * a.ld_v + (int64_t)h * dv + d]);
    }
    __syncthreads();
    for (int t = 0; t < nb; ++t) {
      const float vt = owner ? vs[t * dv + vi] : 0.f;
      const float* kt = ks + t * dkp + si * DPT;
      const float* qt = qs + t * dkp + si * DPT;
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < DPT; ++j) {
        S[j] = fmaf(kt[j], vt, decay * S[j]);
        o = fmaf(S[j], qt[j], o);
      }
      for (int m = 1; m < split; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (owner && si == 0) os[t * dv + vi] = o;
    }
    __syncthreads();
    // a warp per row: the head's output over its root mean square, times silu(gate)
    for (int t = tid >> 5; t < nb; t += nthreads >> 5) {
      const int lane = tid & 31;
      float inv = 1.f;
      if (a.unit_norm) {
        float sq = 0.f;
        for (int c = lane; c < dv; c += 32) sq = fmaf(os[t * dv + c], os[t * dv + c], sq);
        sq = warp_sum(sq);
        inv = 1.0f / sqrtf(sq / (float)dv + a.eps);
      }
      const int64_t row = start + t0 + t;
      for (int c = lane; c < dv; c += 32) {
        float y = os[t * dv + c] * inv;
        if (gate != nullptr) {
          const float g = to_f32(gate[row * a.ld_gate + (int64_t)h * dv + c]);
          y *= g / (1.0f + expf(-g));
        }
        out[row * a.ld_out + (int64_t)h * dv + c] = from_f32<T>(y);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < DPT; ++j) {
    const int d = si * DPT + j;
    if (owner && d < dk) st[(int64_t)d * dv + vi] = S[j];
  }
}

template <typename T, int DPT>
int launch_retention(const RetentionArgs& a, int n_seqs, int threads, cudaStream_t stream) {
  const size_t smem = ((size_t)2 * TB * a.split * DPT + (size_t)2 * TB * a.dv) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(retention_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) KVAD_FAIL(KVAD_ERR_CUDA, "retention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  kvad_launch(retention_kernel<T, DPT>, dim3(n_seqs, a.heads), dim3(threads), smem, stream, a);
  KVAD_CHECK_LAUNCH("retention");
  return KVAD_OK;
}

template <typename T>
int dispatch_retention(RetentionArgs& a, int n_seqs, cudaStream_t stream) {
  // the fewest state entries a thread such that a head's columns times their split fit a block
  for (int dpt : {8, 16, 32, 64}) {
    int split = 1;
    while (split * dpt < a.dk) split <<= 1;
    if (split > 32) continue;
    const int threads = (a.dv * split + 31) / 32 * 32;
    if (threads > max_threads(dpt)) continue;
    a.split = split;
    switch (dpt) {
      case 8: return launch_retention<T, 8>(a, n_seqs, threads, stream);
      case 16: return launch_retention<T, 16>(a, n_seqs, threads, stream);
      case 32: return launch_retention<T, 32>(a, n_seqs, threads, stream);
      default: return launch_retention<T, 64>(a, n_seqs, threads, stream);
    }
  }
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "retention: a state of %d x %d a head does not fit a block (up to 128 x 128, or 64 x 256)", a.dk, a.dv);
}

}  // namespace

KVAD_EXPORT int kvad_retention(int dtype, const void* q, int64_t ld_q, const void* k, int64_t ld_k, const void* v, int64_t ld_v,
                               const void* gate, int64_t ld_gate, void* out, int64_t ld_out, float* state, const int* seq_starts,
                               const int* kv_lens, const int* seq_slots, const float* decay, const float* inv_freq, int rot_dims,
                               int interleaved, int n_seqs, int heads, int dk, int dv, float k_scale, float eps, int unit_norm,
                               cudaStream_t stream) {
  KVAD_REQUIRE(n_seqs >= 0 && heads > 0 && dk > 0 && dv > 0, "retention: bad sizes seqs=%d heads=%d dk=%d dv=%d", n_seqs, heads, dk, dv);
  KVAD_REQUIRE(state != nullptr && decay != nullptr && seq_starts && kv_lens && seq_slots, "retention: needs state, decays and the step's sequences");
  KVAD_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk, "retention: %d rotated entries of %d", rot_dims, dk);
  KVAD_REQUIRE(n_seqs <= 65535 * 32 && heads <= 65535, "retention: %d sequences x %d heads are more than one launch takes", n_seqs, heads);
  if (n_seqs == 0) return KVAD_OK;
  RetentionArgs a;
  a.q = q; a.k = k; a.v = v; a.gate = gate; a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_gate = ld_gate;
  a.out = out; a.ld_out = ld_out; a.state = state; a.seq_starts = seq_starts; a.kv_lens = kv_lens; a.seq_slots = seq_slots;
  a.decay = decay; a.inv_freq = rot_dims > 0 ? inv_freq : nullptr; a.rot_dims = rot_dims; a.interleaved = interleaved;
  a.heads = heads; a.dk = dk; a.dv = dv; a.split = 1; a.k_scale = k_scale; a.eps = eps; a.unit_norm = unit_norm;
  if (dtype == KVAD_DTYPE_F32) return dispatch_retention<float>(a, n_seqs, stream);
  if (dtype == KVAD_DTYPE_BF16) return dispatch_retention<__nv_bfloat16>(a, n_seqs, stream);
  KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "retention: unknown dtype %d", dtype);
}

KVAD_DEFINE_LAST_ERROR()
