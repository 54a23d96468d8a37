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
// values go to dense [T, nkv, d] buffers.
#include "common.cuh"

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

TS_EXPORT int ts_qk_joint_norm_rope_store(const void* qk, int act_dtype, long long ld, void* q_out, void* k_dst, void* v_dst,
                                          const int* slot_mapping, const float* q_w, const float* k_w, float eps, const float* cos_sin,
                                          int rot, int T, int nq, int nkv, int d, void* stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || rot < 0 || rot > d || (rot & 1) || (rot > 0 && cos_sin == nullptr)) return TS_ERR_BAD_ARGUMENT;
  const int n = (nq + nkv) * d;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(qk_joint_norm_rope_store_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)qk, ld, (float*)q_out,
                     (float*)k_dst, (float*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq, nkv, d);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(qk_joint_norm_rope_store_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, (const __nv_bfloat16*)qk, ld,
                     (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst, slot_mapping, q_w, k_w, eps, cos_sin, rot, nq,
                     nkv, d);
  return TS_ERR_BAD_ARGUMENT;
}
