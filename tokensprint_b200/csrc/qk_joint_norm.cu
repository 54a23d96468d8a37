// q/k RMSNorm over the whole projection, rotary position encoding and the store of keys and
// values into the paged cache, for attention layers whose q and k are normed before they are cut
// into heads and whose values are the key projection itself.
//
// Per token, from one row [q | k] of the fused projection (q: nq * d entries, k: nkv * d):
//   q' = q * rsqrt(mean(q^2) + eps) * wq       one mean over all nq * d entries, weight [nq * d]
//   k' = k * rsqrt(mean(k^2) + eps) * wk       likewise over nkv * d entries
//   every head of q' and k' is rotated over its first `rot` entries (entry j with j + rot/2,
//   cosines and sines from the step's table [T, rot/2, 2]), the rest of the head passes,
//   q' goes to q_out, k' to the first pool of the cache by slot, and the row k as it was
//   projected (no norm, no rotation) to the second pool: the layer's values.
// Sums of squares, the factor, the weights and the rotation are float32; one rounding at the store.
//
// One CTA per token.  A slot of -1 skips the stores into the cache; without `slot_mapping` keys and
// values go to dense [T, nkv, d] buffers.  The kernel right below reads the row from device memory
// as it goes (rows too long for shared memory); the staged one after it is what normally runs.
#include "common.cuh"

__device__ __forceinline__ void ts_store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void ts_store_pair(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename TA>
__global__ void qk_joint_norm_rope_store_kernel(const TA* __restrict__ qk, long long ld, TA* __restrict__ q_out, TA* __restrict__ k_dst,
                                                TA* __restrict__ v_dst, const int* __restrict__ slot_mapping,
                                                const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                                const float* __restrict__ cos_sin, int rot, int nq, int nkv, int d) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const TA* row = qk + (size_t)t * ld;
  const int nQ = nq * d, nK = nkv * d, half = rot >> 1;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nQ; i += blockDim.x) {
    const float v = ts_to_float(row[i]);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < nK; i += blockDim.x) {
    const float v = ts_to_float(row[nQ + i]);
    sk += v * v;
  }
  sq = ts_block_sum(sq, scratch);
  sk = ts_block_sum(sk, scratch);
  const float rq = 1.f / sqrtf(sq / (float)nQ + eps), rk = 1.f / sqrtf(sk / (float)nK + eps);
  const float* cs = cos_sin + (size_t)t * half * 2;
  const int slot = slot_mapping ? slot_mapping[t] : t;
  TA* qd = q_out + (size_t)t * nQ;
  for (int i = threadIdx.x; i < nQ + nK; i += blockDim.x) {
    const bool is_q = i < nQ;
    if (!is_q && slot < 0) break;  // i only grows: nothing of k is stored
    const int e = is_q ? i : i - nQ;
    const float* w = is_q ? q_w : k_w;
    const float r = is_q ? rq : rk;
    const int j = e % d;
    const float x = ts_to_float(row[i]) * r * w[e];
    float y = x;
    if (j < half) {
      const float partner = ts_to_float(row[i + half]) * r * w[e + half];
      y = x * cs[2 * j] - partner * cs[2 * j + 1];
    } else if (j < 2 * half) {
      const float partner = ts_to_float(row[i - half]) * r * w[e - half];
      y = x * cs[2 * (j - half)] + partner * cs[2 * (j - half) + 1];
    }
    if (is_q) {
      qd[e] = ts_from_float<TA>(y);
    } else {
      k_dst[(size_t)slot * nK + e] = ts_from_float<TA>(y);
      v_dst[(size_t)slot * nK + e] = row[i];
    }
  }
}

// The same through shared memory, for rows that fit it (every practical size): the row is read
// once with the widest loads its alignment allows and staged with the norm weights already on it,
// the values leave in that first pass, partners of the rotation come from shared memory, and
// q' and k' leave in pairs of elements.
template <typename TA>
__global__ void qk_joint_norm_rope_store_staged_kernel(const TA* __restrict__ qk, long long ld, TA* __restrict__ q_out, TA* __restrict__ k_dst,
                                                       TA* __restrict__ v_dst, const int* __restrict__ slot_mapping,
                                                       const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                                       const float* __restrict__ cos_sin, int rot, int nq, int nkv, int d, int wide) {
  ts_pdl_prologue();
  extern __shared__ float xs[];  // the row [q | k] times its norm weights, float32 (only the factor 1/rms is still missing)
  __shared__ float2 scratch2[33];
  const int t = blockIdx.x;
  const TA* row = qk + (size_t)t * ld;
  const int nQ = nq * d, nK = nkv * d, n = nQ + nK, half = rot >> 1;
  const int slot = slot_mapping ? slot_mapping[t] : t;
  float sq = 0.f, sk = 0.f;
  // First pass: the sums of squares, the row times the weights into shared memory, and the values (the k row as it is)
  // straight to their place: nothing of that waits for the norm.
  if (wide) {  // n, nQ and ld are multiples of 4, the row, the weights and the value pool start on 4-element boundaries
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      float v[4];
      if constexpr (sizeof(TA) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(row + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(row + i);
        v[0] = raw.x, v[1] = raw.y, v[2] = raw.z, v[3] = raw.w;
      }
      const float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
      const bool is_q = i < nQ;
      if (is_q) sq += ss; else sk += ss;
      const float4 w4 = *reinterpret_cast<const float4*>(is_q ? q_w + i : k_w + (i - nQ));
      *reinterpret_cast<float4*>(xs + i) = make_float4(v[0] * w4.x, v[1] * w4.y, v[2] * w4.z, v[3] * w4.w);
      if (!is_q && slot >= 0) {
        TA* vd = v_dst + (size_t)slot * nK + (i - nQ);
        if constexpr (sizeof(TA) == 2) {
          *reinterpret_cast<uint2*>(vd) = *reinterpret_cast<const uint2*>(row + i);
        } else {
          *reinterpret_cast<float4*>(vd) = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = ts_to_float(row[i]);
      const bool is_q = i < nQ;
      if (is_q) sq += v * v; else sk += v * v;
      xs[i] = v * (is_q ? q_w[i] : k_w[i - nQ]);
      if (!is_q && slot >= 0) v_dst[(size_t)slot * nK + (i - nQ)] = row[i];
    }
  }
  {  // both sums of squares in one pass over the block (its barriers also make the staged row visible to all threads)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    sq = ts_warp_sum(sq);
    sk = ts_warp_sum(sk);
    if (lane == 0) scratch2[warp] = make_float2(sq, sk);
    __syncthreads();
    if (warp == 0) {
      float2 v = lane < nwarps ? scratch2[lane] : make_float2(0.f, 0.f);
      v.x = ts_warp_sum(v.x);
      v.y = ts_warp_sum(v.y);
      if (lane == 0) scratch2[32] = v;
    }
    __syncthreads();
    sq = scratch2[32].x;
    sk = scratch2[32].y;
  }
  const float rq = 1.f / sqrtf(sq / (float)nQ + eps), rk = 1.f / sqrtf(sk / (float)nK + eps);
  const float* cs = cos_sin + (size_t)t * half * 2;
  auto element = [&](int i, int j) -> float {  // entry i of [q' | k'], which is entry j of its head
    const float r = i < nQ ? rq : rk;
    const float x = xs[i] * r;
    if (j < half) return x * cs[2 * j] - xs[i + half] * r * cs[2 * j + 1];
    if (j < 2 * half) return x * cs[2 * (j - half)] + xs[i - half] * r * cs[2 * (j - half) + 1];
    return x;
  };
  TA* qd = q_out + (size_t)t * nQ;
  const int stop = slot < 0 ? nQ : n;  // a token without a slot stores nothing of k
  if ((d & 1) == 0 && ((uintptr_t)q_out & 7) == 0 && ((uintptr_t)k_dst & 7) == 0) {
    // a thread's place inside a head moves by the same amount every round: no division in the loop
    const int step = (blockDim.x * 2) % d;
    int j = (threadIdx.x * 2) % d;
    for (int i = threadIdx.x * 2; i < stop; i += blockDim.x * 2) {  // nQ and nK are even: a pair never straddles q and k, nor two heads
      const float a = element(i, j), b = element(i + 1, j + 1);
      j += step;
      if (j >= d) j -= d;
      if (i < nQ) {
        ts_store_pair(qd + i, a, b);
      } else {
        ts_store_pair(k_dst + (size_t)slot * nK + (i - nQ), a, b);
      }
    }
  } else {
    for (int i = threadIdx.x; i < stop; i += blockDim.x) {
      const float a = element(i, i % d);
      if (i < nQ) {
        qd[i] = ts_from_float<TA>(a);
      } else {
        k_dst[(size_t)slot * nK + (i - nQ)] = ts_from_float<TA>(a);
      }
    }
  }
}

TS_EXPORT int ts_qk_joint_norm_rope_store(const void* qk, int act_dtype, long long ld, void* q_out, void* k_dst, void* v_dst,
                                          const int* slot_mapping, const float* q_w, const float* k_w, float eps, const float* cos_sin,
                                          int rot, int T, int nq, int nkv, int d, void* stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || rot < 0 || rot > d || (rot & 1) || (rot > 0 && cos_sin == nullptr)) return TS_ERR_BAD_ARGUMENT;
  const int n = (nq + nkv) * d;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)n * sizeof(float);
  if (smem <= 40 * 1024) {
    const size_t elem = act_dtype == TS_DTYPE_F32 ? 4 : 2;
    const int wide = (n % 4 == 0 && (nq * d) % 4 == 0 && ld % 4 == 0 && ((uintptr_t)qk % (4 * elem)) == 0 && ((uintptr_t)v_dst % (4 * elem)) == 0 &&
                      (((uintptr_t)q_w | (uintptr_t)k_w) % 16) == 0) ? 1 : 0;
    // Few tokens: a row's pieces spread over many threads (shortest latency).  Many: smaller CTAs (16 entries a thread), so that
    // an SM holds more tokens at once and one token's load, reduction and store phases overlap with the others'.
    const int th = T >= 512 ? min(512, max(128, (n / 16 + 31) / 32 * 32)) : (wide ? min(512, max(64, (n / 4 + 31) / 32 * 32)) : threads);
    if (act_dtype == TS_DTYPE_F32)
      return ts_launch(qk_joint_norm_rope_store_staged_kernel<float>, dim3(T), dim3(th), smem, s, (const float*)qk, ld, (float*)q_out,
                       (float*)k_dst, (float*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq, nkv, d, wide);
    if (act_dtype == TS_DTYPE_BF16)
      return ts_launch(qk_joint_norm_rope_store_staged_kernel<__nv_bfloat16>, dim3(T), dim3(th), smem, s, (const __nv_bfloat16*)qk, ld,
                       (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq,
                       nkv, d, wide);
    return TS_ERR_BAD_ARGUMENT;
  }
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(qk_joint_norm_rope_store_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)qk, ld, (float*)q_out,
                     (float*)k_dst, (float*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq, nkv, d);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(qk_joint_norm_rope_store_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, (const __nv_bfloat16*)qk, ld,
                     (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq,
                     nkv, d);
  return TS_ERR_BAD_ARGUMENT;
}
