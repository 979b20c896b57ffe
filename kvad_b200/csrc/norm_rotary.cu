// Row-wise kernels of designs with RMS norms, rotary positions and gated activations.
// All arithmetic is 32-bit (sums of squares, angles, sines, gates); the element type only says how
// tensors are stored.
//
//   rmsnorm           y = x / sqrt(mean(x^2) + eps) * w      (w absent: 1; `unit_offset`: 1 + w)
//   residual_rmsnorm  x += mult * delta; delta = 0; y = rmsnorm(x)   - a block whose sublayers add into `delta`
//                     leaves the scaled sum to the next reader of the stream
//   rotary            pairs of a head's first `dims` entries turned by position * base^(-2i/dims), either
//                     entry i with i + dims/2 ("half") or 2i with 2i + 1 ("interleaved")
//   gate_mul          out = act(a) * b,  act = silu or sigmoid
//   scale_add         x += mult * delta; delta = 0
#include "common.cuh"

using namespace kvad;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// A block of 128 threads per row.  Two passes over the row (the second finds it in the L1), four entries a thread
// and trip where the row allows 16-byte loads of 32-bit values: few trips, their loads in flight together.  The
// sums run thread by thread in column order, then a shuffle tree and the warps in order - a row's bits do not
// depend on its company.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
rmsnorm_kernel(const TI* __restrict__ x, int64_t ld_in, const int* __restrict__ row_index, const void* __restrict__ w,
               int w_f32, int unit_offset, TO* __restrict__ out, int64_t ld_out, int n_rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const TI* xr = x + (int64_t)(row_index ? row_index[r] : r) * ld_in;
  float sq = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    const float v = to_f32(xr[c]);
    sq = fmaf(v, v, sq);
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
  TO* o = out + (int64_t)r * ld_out;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += 128) {
    float g = 1.f;
    if (w != nullptr) g = load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f);
    o[c] = from_f32<TO>(to_f32(xr[c]) * inv * g);
  }
}

// The same on the 32-bit residual stream with a pending scaled sum: v = x + mult * delta.  With `write_back`
// (all rows are walked) v replaces x and delta is cleared for the sublayers of the next block; with a row
// list (the head reads a few rows) nothing is written back.  `vec`: the width is a multiple of 4 and the rows
// start on 16-byte boundaries.
template <typename TO>
__global__ void __launch_bounds__(128)
residual_rmsnorm_kernel(float* __restrict__ x, float* __restrict__ delta, float mult, int write_back,
                        const int* __restrict__ row_index, const void* __restrict__ w, int w_f32, int unit_offset,
                        TO* __restrict__ out, int64_t ld_out, int n_rows, int width, float eps, int vec) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int64_t src = (int64_t)(row_index ? row_index[r] : r) * width;
  float* xr = x + src;
  float* dr = delta + src;
  float sq = 0.f;
  if (vec) {
#pragma unroll 2
    for (int c = threadIdx.x * 4; c < width; c += 512) {
      const float4 xv = *reinterpret_cast<const float4*>(xr + c), dv = *reinterpret_cast<const float4*>(dr + c);
      const float4 v = make_float4(fmaf(mult, dv.x, xv.x), fmaf(mult, dv.y, xv.y), fmaf(mult, dv.z, xv.z), fmaf(mult, dv.w, xv.w));
      if (write_back) {
        *reinterpret_cast<float4*>(xr + c) = v;
        *reinterpret_cast<float4*>(dr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += 128) {
      const float v = fmaf(mult, dr[c], xr[c]);
      if (write_back) {
        xr[c] = v;
        dr[c] = 0.f;
      }
      sq = fmaf(v, v, sq);
    }
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)width + eps);
  TO* o = out + (int64_t)r * ld_out;
  const int step = vec ? 4 : 1;
  for (int c0 = threadIdx.x * step; c0 < width; c0 += 128 * step) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = c0 + e;
      if (e < step) {
        const float v = write_back ? xr[c] : fmaf(mult, dr[c], xr[c]);     // (the thread reads what it wrote)
        float g = 1.f;
        if (w != nullptr) g = load_param(w, c, w_f32) + (unit_offset ? 1.f : 0.f);
        o[c] = from_f32<TO>(v * inv * g);
      }
    }
  }
}

__global__ void scale_add_kernel(float* __restrict__ x, float* __restrict__ delta, float mult, int64_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    x[i] = fmaf(mult, delta[i], x[i]);
    delta[i] = 0.f;
  }
}

// One thread per (row, head, pair).  `src` and `dst` may be the same buffer (each pair is read, then written, by
// one thread) or different ones (a copy that rotates).
template <typename T>
__global__ void rotary_kernel(const T* __restrict__ src, int64_t ld_src, int head_stride_src, int off_src,
                              T* __restrict__ dst, int64_t ld_dst, int head_stride_dst, int off_dst,
                              const int* __restrict__ row_pos, const float* __restrict__ inv_freq, int n_rows, int n_heads,
                              int dims, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = dims / 2;
  const int64_t total = (int64_t)n_rows * n_heads * half;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int p = (int)(i % half), h = (int)((i / half) % n_heads), r = (int)(i / ((int64_t)half * n_heads));
    const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
    const T* s = src + (int64_t)r * ld_src + (int64_t)h * head_stride_src + off_src;
    T* d = dst + (int64_t)r * ld_dst + (int64_t)h * head_stride_dst + off_dst;
    float sn, cs;
    sincosf((float)row_pos[r] * inv_freq[p], &sn, &cs);
    const float u = to_f32(s[a]), v = to_f32(s[b]);
    d[a] = from_f32<T>(u * cs - v * sn);
    d[b] = from_f32<T>(v * cs + u * sn);
  }
}

template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, int64_t ld_a, const T* __restrict__ b, int64_t ld_b,
                                T* __restrict__ out, int64_t ld_out, int n_rows, int width, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = (int64_t)n_rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    const float g = to_f32(a[(int64_t)r * ld_a + c]);
    const float v = to_f32(b[(int64_t)r * ld_b + c]);
    out[(int64_t)r * ld_out + c] = from_f32<T>((act == 0 ? silu_f(g) : sigmoid_f(g)) * v);
  }
}

inline int flat_blocks(int64_t total, int threads) {
  const int64_t b = (total + threads - 1) / threads;
  return (int)(b < 148 * 16 ? b : 148 * 16);
}

}  // namespace

// in_dtype: the element type of `x` (the 32-bit residual stream, or activations of the compute dtype).
KVAD_EXPORT int kvad_rmsnorm(int in_dtype, int out_dtype, const void* x, int64_t ld_in, const int* row_index, const void* w,
                             int w_f32, int unit_offset, void* out, int64_t ld_out, int n_rows, int width, float eps,
                             cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && ld_in >= width && ld_out >= width, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
#define KVAD_RMS(TI, TO)                                                                                                  \
  kvad_launch(rmsnorm_kernel<TI, TO>, grid, block, 0, stream, (const TI*)x, ld_in, row_index, w, w_f32, unit_offset, (TO*)out, \
              ld_out, n_rows, width, eps)
  if (in_dtype == KVAD_DTYPE_F32 && out_dtype == KVAD_DTYPE_F32) KVAD_RMS(float, float);
  else if (in_dtype == KVAD_DTYPE_F32 && out_dtype == KVAD_DTYPE_BF16) KVAD_RMS(float, __nv_bfloat16);
  else if (in_dtype == KVAD_DTYPE_BF16 && out_dtype == KVAD_DTYPE_BF16) KVAD_RMS(__nv_bfloat16, __nv_bfloat16);
  else KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "rmsnorm: no form for input dtype %d and output dtype %d", in_dtype, out_dtype);
#undef KVAD_RMS
  KVAD_CHECK_LAUNCH("rmsnorm");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_residual_rmsnorm(int out_dtype, float* x, float* delta, float mult, int write_back, const int* row_index,
                                      const void* w, int w_f32, int unit_offset, void* out, int64_t ld_out, int n_rows,
                                      int width, float eps, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && ld_out >= width && x != nullptr && delta != nullptr, "residual_rmsnorm: bad arguments");
  KVAD_REQUIRE(!(write_back && row_index), "residual_rmsnorm: writing back goes with walking all rows");
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(n_rows), block(128);
  const int vec = (width % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta)) & 15) == 0) ? 1 : 0;
  if (out_dtype == KVAD_DTYPE_F32)
    kvad_launch(residual_rmsnorm_kernel<float>, grid, block, 0, stream, x, delta, mult, write_back, row_index, w, w_f32, unit_offset,
                (float*)out, ld_out, n_rows, width, eps, vec);
  else if (out_dtype == KVAD_DTYPE_BF16)
    kvad_launch(residual_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, x, delta, mult, write_back, row_index, w, w_f32,
                unit_offset, (__nv_bfloat16*)out, ld_out, n_rows, width, eps, vec);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "residual_rmsnorm: unknown dtype %d", out_dtype);
  KVAD_CHECK_LAUNCH("residual_rmsnorm");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_scale_add(float* x, float* delta, float mult, int64_t total, cudaStream_t stream) {
  KVAD_REQUIRE(total >= 0 && x != nullptr && delta != nullptr, "scale_add: bad arguments");
  if (total == 0) return KVAD_OK;
  kvad_launch(scale_add_kernel, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, x, delta, mult, total);
  KVAD_CHECK_LAUNCH("scale_add");
  return KVAD_OK;
}

KVAD_EXPORT int kvad_rotary(int dtype, const void* src, int64_t ld_src, int head_stride_src, int off_src, void* dst,
                            int64_t ld_dst, int head_stride_dst, int off_dst, const int* row_pos, const float* inv_freq,
                            int n_rows, int n_heads, int dims, int interleaved, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && n_heads > 0 && dims > 0 && dims % 2 == 0, "rotary: bad sizes rows=%d heads=%d dims=%d", n_rows, n_heads, dims);
  KVAD_REQUIRE(row_pos != nullptr && inv_freq != nullptr, "rotary: needs positions and frequencies");
  if (n_rows == 0) return KVAD_OK;
  const int64_t total = (int64_t)n_rows * n_heads * (dims / 2);
  dim3 grid(flat_blocks(total, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(rotary_kernel<float>, grid, block, 0, stream, (const float*)src, ld_src, head_stride_src, off_src, (float*)dst, ld_dst,
                head_stride_dst, off_dst, row_pos, inv_freq, n_rows, n_heads, dims, interleaved);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(rotary_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)src, ld_src, head_stride_src, off_src,
                (__nv_bfloat16*)dst, ld_dst, head_stride_dst, off_dst, row_pos, inv_freq, n_rows, n_heads, dims, interleaved);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "rotary: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("rotary");
  return KVAD_OK;
}

// act: 0 = silu, 1 = sigmoid.
KVAD_EXPORT int kvad_gate_mul(int dtype, const void* a, int64_t ld_a, const void* b, int64_t ld_b, void* out, int64_t ld_out,
                              int n_rows, int width, int act, cudaStream_t stream) {
  KVAD_REQUIRE(n_rows >= 0 && width > 0 && (act == 0 || act == 1), "gate_mul: bad arguments rows=%d width=%d act=%d", n_rows, width, act);
  if (n_rows == 0) return KVAD_OK;
  dim3 grid(flat_blocks((int64_t)n_rows * width, 256)), block(256);
  if (dtype == KVAD_DTYPE_F32)
    kvad_launch(gate_mul_kernel<float>, grid, block, 0, stream, (const float*)a, ld_a, (const float*)b, ld_b, (float*)out, ld_out, n_rows, width, act);
  else if (dtype == KVAD_DTYPE_BF16)
    kvad_launch(gate_mul_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)a, ld_a, (const __nv_bfloat16*)b, ld_b,
                (__nv_bfloat16*)out, ld_out, n_rows, width, act);
  else
    KVAD_FAIL(KVAD_ERR_UNSUPPORTED, "gate_mul: unknown dtype %d", dtype);
  KVAD_CHECK_LAUNCH("gate_mul");
  return KVAD_OK;
}

KVAD_DEFINE_LAST_ERROR()
