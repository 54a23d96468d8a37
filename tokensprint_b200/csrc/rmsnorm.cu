// Residual add + RMSNorm over the float32 residual stream.
//
//   h = hidden[row] (+ delta[row]);  hidden[row] = h (when a delta was added);
//   out[r] = h * rsqrt(mean(h^2) + eps) * weight
//
// Sums, mean, rsqrt and the scaling are float32 with one rounding at the store, as in the
// reference's kernel (engine/kernels/triton/rmsnorm.py:19-42); the residual sum is float32
// too (the reference adds in the model dtype, engine/nn/layers.py:112,121).  With
// `row_index` the kernel reads only the listed rows (the rows whose logits are wanted
// before the final norm) and leaves `hidden` untouched.
#include "common.cuh"

template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, TA* __restrict__ out,
                                   const int* __restrict__ row_index, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = row_index ? row_index[r] : r;
  float* h = hidden + (size_t)row * H;
  const TA* d = delta ? delta + (size_t)row * H : nullptr;
  TA* o = out + (size_t)r * H;
  const bool write_back = (d != nullptr) && (row_index == nullptr);

  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (d) v += ts_to_float(d[i]);
    if (write_back) h[i] = v;
    ss += v * v;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (d && !write_back) v += ts_to_float(d[i]);
    o[i] = ts_from_float<TA>(v * rstd * weight[i]);
  }
}

// Fast path for widths that are a multiple of 4: every thread keeps its (up to
// RN_MAX_CHUNKS) float4 pieces of the row in registers between the two passes, so the row
// is read once, with 16-byte loads issued back to back.
#define RN_MAX_CHUNKS 4

__device__ __forceinline__ float4 ts_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ts_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void ts_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ts_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TA>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ hidden, const TA* __restrict__ delta,
                                       const float* __restrict__ weight, TA* __restrict__ out,
                                       const int* __restrict__ row_index, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = row_index ? row_index[r] : r;
  float* h = hidden + (size_t)row * H;
  const TA* d = delta ? delta + (size_t)row * H : nullptr;
  TA* o = out + (size_t)r * H;
  const bool write_back = (d != nullptr) && (row_index == nullptr);
  const int chunks = H >> 2;
  float4 v[RN_MAX_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      v[k] = ts_load4(h + 4 * c);
      if (d) {
        const float4 dv = ts_load4(d + 4 * c);
        v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      if (write_back) ts_store4(h + 4 * c, v[k]);
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      const float4 w = ts_load4(weight + 4 * c);
      ts_store4(o + 4 * c, make_float4(v[k].x * rstd * w.x, v[k].y * rstd * w.y, v[k].z * rstd * w.z, v[k].w * rstd * w.w));
    }
  }
}

template <typename TA>
static int launch_add_rmsnorm(float* hidden, const void* delta, const float* weight, void* out,
                              const int* row_index, int rows, int H, float eps, cudaStream_t s) {
  const int chunks = H >> 2;
  const bool aligned = (H % 4 == 0) && (((uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) % 16 == 0);
  if (aligned && chunks <= RN_MAX_CHUNKS * 1024) {
    int threads = (chunks + RN_MAX_CHUNKS - 1) / RN_MAX_CHUNKS;
    if (rows <= 512) threads = chunks;  // few rows: one piece per thread, shortest latency
    threads = min(1024, max(32, (threads + 31) / 32 * 32));
    return ts_launch(add_rmsnorm_vec_kernel<TA>, dim3(rows), dim3(threads), 0, s, hidden, (const TA*)delta, weight, (TA*)out, row_index, H, eps);
  } else {
    int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64));
    return ts_launch(add_rmsnorm_kernel<TA>, dim3(rows), dim3(threads), 0, s, hidden, (const TA*)delta, weight, (TA*)out, row_index, H, eps);
  }
}

TS_EXPORT int ts_add_rmsnorm(float* hidden, const void* delta, int act_dtype, const float* weight,
                             void* out, const int* row_index, int rows, int H, float eps,
                             void* stream) {
  if (rows <= 0) return 0;
  if (H <= 0) return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return launch_add_rmsnorm<float>(hidden, delta, weight, out, row_index, rows, H, eps, s);
  if (act_dtype == TS_DTYPE_BF16)
    return launch_add_rmsnorm<__nv_bfloat16>(hidden, delta, weight, out, row_index, rows, H, eps, s);
  return TS_ERR_BAD_ARGUMENT;
}

// hidden[row] += delta[row] without a norm (the last residual sum when nothing follows it).
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ hidden, const TA* __restrict__ delta, size_t n) {
  ts_pdl_prologue();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += ts_to_float(delta[i]);
}

TS_EXPORT int ts_residual_add(float* hidden, const void* delta, int act_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, s, hidden, (const float*)delta, (size_t)n);
  else if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(residual_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, hidden, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}

// The norm on a branch's output, for layers that norm what a sublayer returns instead of what it
// reads:  hidden[row] += branch[row] * rsqrt(mean(branch[row]^2) + eps) * weight, all in float32,
// and, if asked for, the new row once more in the compute type (what the next sublayer reads).
template <typename TB, typename TO>
__global__ void rmsnorm_add_kernel(const TB* __restrict__ branch, const float* __restrict__ weight, float* __restrict__ hidden,
                                   TO* __restrict__ rounded, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const TB* b = branch + (size_t)row * H;
  float* h = hidden + (size_t)row * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = ts_to_float(b[i]);
    ss += v * v;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = h[i] + ts_to_float(b[i]) * rstd * weight[i];
    h[i] = v;
    if (rounded) rounded[(size_t)row * H + i] = ts_from_float<TO>(v);
  }
}

// The same for widths that are a multiple of 4: the branch row and the stream's row stay in
// registers between the sum of squares and the update, so each is read once, with 16-byte loads
// issued back to back.
template <typename TB, typename TO>
__global__ void rmsnorm_add_vec_kernel(const TB* __restrict__ branch, const float* __restrict__ weight, float* __restrict__ hidden,
                                       TO* __restrict__ rounded, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const TB* b = branch + (size_t)row * H;
  float* h = hidden + (size_t)row * H;
  const int chunks = H >> 2;
  float4 bv[RN_MAX_CHUNKS], hv[RN_MAX_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      bv[k] = ts_load4(b + 4 * c);
      hv[k] = ts_load4(h + 4 * c);
    }
  }
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) ss += bv[k].x * bv[k].x + bv[k].y * bv[k].y + bv[k].z * bv[k].z + bv[k].w * bv[k].w;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      const float4 w = ts_load4(weight + 4 * c);
      const float4 v = make_float4(hv[k].x + bv[k].x * rstd * w.x, hv[k].y + bv[k].y * rstd * w.y, hv[k].z + bv[k].z * rstd * w.z,
                                   hv[k].w + bv[k].w * rstd * w.w);
      ts_store4(h + 4 * c, v);
      if (rounded) ts_store4(rounded + (size_t)row * H + 4 * c, v);
    }
  }
}

template <typename TB, typename TO>
static int launch_rmsnorm_add(const void* branch, const float* weight, float* hidden, void* rounded, int rows, int H, float eps, cudaStream_t s) {
  const int chunks = H >> 2;
  const bool aligned = (H % 4 == 0) && (((uintptr_t)branch | (uintptr_t)weight | (uintptr_t)hidden | (uintptr_t)rounded) % 16 == 0);
  if (aligned && chunks <= RN_MAX_CHUNKS * 1024) {
    int threads = (chunks + RN_MAX_CHUNKS - 1) / RN_MAX_CHUNKS;
    if (rows <= 512) threads = chunks;  // few rows: one piece per thread, shortest latency
    threads = min(1024, max(32, (threads + 31) / 32 * 32));
    return ts_launch(rmsnorm_add_vec_kernel<TB, TO>, dim3(rows), dim3(threads), 0, s, (const TB*)branch, weight, hidden, (TO*)rounded, H, eps);
  }
  const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64));
  return ts_launch(rmsnorm_add_kernel<TB, TO>, dim3(rows), dim3(threads), 0, s, (const TB*)branch, weight, hidden, (TO*)rounded, H, eps);
}

TS_EXPORT int ts_rmsnorm_add(const void* branch, int branch_dtype, const float* weight, float* hidden, void* rounded, int rounded_dtype,
                             int rows, int H, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (H <= 0) return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  if (branch_dtype == TS_DTYPE_F32 && (rounded == nullptr || rounded_dtype == TS_DTYPE_F32))
    return launch_rmsnorm_add<float, float>(branch, weight, hidden, rounded, rows, H, eps, s);
  if (branch_dtype == TS_DTYPE_F32 && rounded_dtype == TS_DTYPE_BF16)
    return launch_rmsnorm_add<float, __nv_bfloat16>(branch, weight, hidden, rounded, rows, H, eps, s);
  if (branch_dtype == TS_DTYPE_BF16 && (rounded == nullptr || rounded_dtype == TS_DTYPE_BF16))
    return launch_rmsnorm_add<__nv_bfloat16, __nv_bfloat16>(branch, weight, hidden, rounded, rows, H, eps, s);
  return TS_ERR_BAD_ARGUMENT;
}

// out = rows in another element type (what a sublayer that reads the residual stream itself is
// handed when nothing before it has produced the rounded rows; or rounded rows widened again).
template <typename TI, typename TO>
__global__ void round_rows_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  ts_pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = ts_from_float<TO>(ts_to_float(in[i]));
}

TS_EXPORT int ts_round_rows(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_BF16)
    return ts_launch(round_rows_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const float*)in, (__nv_bfloat16*)out, (size_t)n);
  if (in_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_F32)
    return ts_launch(round_rows_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)in, (float*)out, (size_t)n);
  if (in_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_F32)
    return ts_launch(round_rows_kernel<float, float>, dim3(blocks), dim3(256), 0, s, (const float*)in, (float*)out, (size_t)n);
  return TS_ERR_BAD_ARGUMENT;
}

// A sublayer between two norms, with a learned scale per channel on its way back into the stream:
//   hidden[row] += branch[row] * rsqrt(mean(branch[row]^2) + eps) * weight * scale      (scale may be absent)
// and, if the next norm's weight is given, that norm on the new row in the same pass:
//   out[row] = hidden[row] * rsqrt(mean(hidden[row]^2) + next_eps) * next_weight
// All sums and the stream in float32; `out` in the compute type.  One CTA per row; the row stays in
// registers between the two sums of squares where it is short enough, else it is read again.
#define BN_KEEP 8  // elements a thread keeps between the passes
template <typename TB, typename TO>
__global__ void branch_norm_add_kernel(const TB* __restrict__ branch, const float* __restrict__ weight, const float* __restrict__ scale,
                                       float* __restrict__ hidden, const float* __restrict__ next_weight, TO* __restrict__ out, int H,
                                       float eps, float next_eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const TB* b = branch + (size_t)row * H;
  float* h = hidden + (size_t)row * H;
  const bool keep = H <= BN_KEEP * (int)blockDim.x;
  float kept[BN_KEEP];
  float ss = 0.f;
  for (int i = threadIdx.x, n = 0; i < H; i += blockDim.x, ++n) {
    const float v = ts_to_float(b[i]);
    if (keep && n < BN_KEEP) kept[n] = v;
    ss += v * v;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)H + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x, n = 0; i < H; i += blockDim.x, ++n) {
    const float bv = (keep && n < BN_KEEP) ? kept[n] : ts_to_float(b[i]);
    float add = bv * rstd * weight[i];
    if (scale) add *= scale[i];
    const float v = h[i] + add;
    h[i] = v;
    if (keep && n < BN_KEEP) kept[n] = v;
    ss2 += v * v;
  }
  if (next_weight == nullptr) return;
  ss2 = ts_block_sum(ss2, scratch);
  const float rstd2 = 1.f / sqrtf(ss2 / (float)H + next_eps);
  for (int i = threadIdx.x, n = 0; i < H; i += blockDim.x, ++n) {
    const float v = (keep && n < BN_KEEP) ? kept[n] : h[i];
    out[(size_t)row * H + i] = ts_from_float<TO>(v * rstd2 * next_weight[i]);
  }
}

// The same for widths that are a multiple of 4 (up to RN_MAX_CHUNKS * 4096): the branch row and the
// stream's row stay in registers from the first sum of squares to the last store, every access is
// 8 or 16 bytes wide and the loads are issued back to back.
template <typename TB, typename TO>
__global__ void branch_norm_add_vec_kernel(const TB* __restrict__ branch, const float* __restrict__ weight, const float* __restrict__ scale,
                                           float* __restrict__ hidden, const float* __restrict__ next_weight, TO* __restrict__ out, int H,
                                           float eps, float next_eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const TB* b = branch + (size_t)row * H;
  float* h = hidden + (size_t)row * H;
  const int chunks = H >> 2;
  float4 bv[RN_MAX_CHUNKS], hv[RN_MAX_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      bv[k] = ts_load4(b + 4 * c);
      hv[k] = ts_load4(h + 4 * c);
    }
  }
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) ss += bv[k].x * bv[k].x + bv[k].y * bv[k].y + bv[k].z * bv[k].z + bv[k].w * bv[k].w;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)H + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      const float4 w = ts_load4(weight + 4 * c);
      float4 add = make_float4(bv[k].x * rstd * w.x, bv[k].y * rstd * w.y, bv[k].z * rstd * w.z, bv[k].w * rstd * w.w);
      if (scale) {
        const float4 sc = ts_load4(scale + 4 * c);
        add = make_float4(add.x * sc.x, add.y * sc.y, add.z * sc.z, add.w * sc.w);
      }
      hv[k] = make_float4(hv[k].x + add.x, hv[k].y + add.y, hv[k].z + add.z, hv[k].w + add.w);
      ts_store4(h + 4 * c, hv[k]);
      ss2 += hv[k].x * hv[k].x + hv[k].y * hv[k].y + hv[k].z * hv[k].z + hv[k].w * hv[k].w;
    }
  }
  if (next_weight == nullptr) return;
  ss2 = ts_block_sum(ss2, scratch);
  const float rstd2 = 1.f / sqrtf(ss2 / (float)H + next_eps);
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      const float4 w = ts_load4(next_weight + 4 * c);
      ts_store4(out + (size_t)row * H + 4 * c, make_float4(hv[k].x * rstd2 * w.x, hv[k].y * rstd2 * w.y, hv[k].z * rstd2 * w.z, hv[k].w * rstd2 * w.w));
    }
  }
}

template <typename TB, typename TO>
static int launch_branch_norm_add(const void* branch, const float* weight, const float* scale, float* hidden, const float* next_weight, void* out,
                                  int rows, int H, float eps, float next_eps, cudaStream_t s) {
  const int chunks = H >> 2;
  const bool aligned = (H % 4 == 0) && (((uintptr_t)branch | (uintptr_t)weight | (uintptr_t)scale | (uintptr_t)hidden | (uintptr_t)next_weight |
                                         (uintptr_t)out) % 16 == 0);
  if (aligned && chunks <= RN_MAX_CHUNKS * 1024) {
    int threads = (chunks + RN_MAX_CHUNKS - 1) / RN_MAX_CHUNKS;
    if (rows <= 512) threads = chunks;  // few rows: one piece per thread, shortest latency
    threads = min(1024, max(32, (threads + 31) / 32 * 32));
    return ts_launch(branch_norm_add_vec_kernel<TB, TO>, dim3(rows), dim3(threads), 0, s, (const TB*)branch, weight, scale, hidden, next_weight,
                     (TO*)out, H, eps, next_eps);
  }
  const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64));
  return ts_launch(branch_norm_add_kernel<TB, TO>, dim3(rows), dim3(threads), 0, s, (const TB*)branch, weight, scale, hidden, next_weight,
                   (TO*)out, H, eps, next_eps);
}

TS_EXPORT int ts_branch_norm_add(const void* branch, int branch_dtype, const float* weight, const float* scale, float* hidden,
                                 const float* next_weight, void* out, int out_dtype, int rows, int H, float eps, float next_eps,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || (next_weight != nullptr && out == nullptr)) return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  if (next_weight == nullptr) out_dtype = branch_dtype;
  if (branch_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_F32)
    return launch_branch_norm_add<float, float>(branch, weight, scale, hidden, next_weight, out, rows, H, eps, next_eps, s);
  if (branch_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_BF16)
    return launch_branch_norm_add<__nv_bfloat16, __nv_bfloat16>(branch, weight, scale, hidden, next_weight, out, rows, H, eps, next_eps, s);
  return TS_ERR_BAD_ARGUMENT;
}

// hidden[row] += rows[row] (if given) + vector (if given), float32: what a model adds to the stream
// between two runs of layers (the embedding rows once more, a learned vector per pass).
__global__ void stream_add_kernel(float* __restrict__ hidden, const float* __restrict__ rows, const float* __restrict__ vector, int H,
                                  size_t n) {
  ts_pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = hidden[i];
  if (rows) v += rows[i];
  if (vector) v += vector[i % H];
  hidden[i] = v;
}

TS_EXPORT int ts_stream_add(float* hidden, const float* rows, const float* vector, int T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0) return TS_ERR_BAD_ARGUMENT;
  const size_t n = (size_t)T * H;
  return ts_launch(stream_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, hidden, rows, vector, H, n);
}
