// Latent attention on the tensor cores (bfloat16, mma.sync m16n8k16, float32 sums), compiled for
// one pair of sizes: TS_LAT_RANK latent entries and TS_LAT_ROT rotated key entries per cached row
// (both multiples of 16).  Prompt portions and decode steps run the same kernel.
//
// Every head of a token scores the same cached rows, so the (token, head) pairs of one sequence
// are simply the rows of a matrix Q [tokens * heads, rank + rot] (the absorbed queries), and a
// cached row serves as key over all its entries and as value over its first `rank`.  A CTA takes
// 32 such rows (two groups of 16) and walks the visible keys in blocks of 64, each block copied
// once into shared memory (16-byte cp.async, two buffers) and used for both products:
//
//   S = Q K^T : the four warps of a row group take 16 keys each, all rank + rot entries;
//   softmax    : running max and sum per row in float32, exchanged between the four warps through
//                shared memory; P is rounded to bfloat16 into shared memory;
//   O += P V   : the four warps take a quarter of the latent's columns each, all 64 keys,
//                so a warp never holds more than 16 x rank/4 sums (a row of 512 entries would
//                not fit one warp's registers).
//
// Decode steps have few rows per sequence; their keys are cut into `splits` ranges, one CTA each
// (grid z), that leave unnormalised sums with their max and sum in scratch, and a second kernel
// merges them.  Keys outside [position - window + 1, position] are masked per row; rows that are
// not copied (outside the visible range, whose pages may be gone) are zeros in shared memory.
// A query's sums depend on its own keys and on the split count only.
#include "../common.cuh"

#ifndef TS_LAT_RANK
#error "compile with -DTS_LAT_RANK=<latent entries> -DTS_LAT_ROT=<rotated entries>"
#endif

namespace {

constexpr int RANK = TS_LAT_RANK, ROT = TS_LAT_ROT, D = RANK + ROT;
constexpr int DS = D + 8;  // shared-memory row stride in elements: an odd number of 16-byte units, so ldmatrix rows fall on different banks
constexpr int BM = 32, BN = 64, THREADS = 256;
constexpr int PS = BN + 8;
constexpr int VT = RANK / 8;         // 8-column tiles of the value side
constexpr int VT_W = (VT + 3) / 4;   // per warp of a row group
static_assert(RANK % 16 == 0 && ROT % 16 == 0 && RANK > 0, "sizes must be multiples of 16");

constexpr size_t SMEM_Q = (size_t)BM * DS * 2, SMEM_K = (size_t)2 * BN * DS * 2, SMEM_P = (size_t)2 * 16 * PS * 2;
constexpr size_t SMEM_STAT = (size_t)2 * 2 * 4 * 16 * 4;
constexpr size_t SMEM_BYTES = SMEM_Q + SMEM_K + SMEM_P + SMEM_STAT;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void group_barrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

__global__ void __launch_bounds__(THREADS, 1) latent_attention_mma_kernel(
    const __nv_bfloat16* __restrict__ q_abs, const __nv_bfloat16* __restrict__ cache, __nv_bfloat16* __restrict__ out,
    const float* __restrict__ gates, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
    const int* __restrict__ block_table, int max_blocks, int page, int H, float scale_log2, int window, int splits,
    float* __restrict__ part_o, float* __restrict__ part_m, float* __restrict__ part_l, long long total_rows) {
  ts_pdl_prologue();
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + SMEM_Q);
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(smem + SMEM_Q + SMEM_K);
  float* smax = reinterpret_cast<float*>(smem + SMEM_Q + SMEM_K + SMEM_P);  // [group][warp][16]
  float* ssum = smax + 2 * 4 * 16;

  const int b = blockIdx.y, split = blockIdx.z;
  const int q0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - q0;
  const int rows_b = qlen * H;
  // the last row tiles of a sequence see the most keys: they are launched first
  const int r0 = ((rows_b + BM - 1) / BM - 1 - (int)blockIdx.x) * BM;
  if (r0 < 0) return;
  const int pos0 = context_lens[b] - qlen;  // position of the sequence's first token of this step
  const int t_lo = r0 / H, t_hi = (min(rows_b, r0 + BM) - 1) / H;
  const int k_hi = pos0 + t_hi;
  const int k_lo = window > 0 ? max(0, pos0 + t_lo - window + 1) : 0;
  const int blk_lo = k_lo / BN, blk_hi = k_hi / BN;
  const int per = (blk_hi - blk_lo + 1 + splits - 1) / splits;
  const int my_lo = blk_lo + split * per, my_hi = min(blk_hi, my_lo + per - 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp >> 2, vq = warp & 3;  // row group, and which quarter of the keys / of the value columns
  const int quad = lane >> 2, qi = lane & 3;
  const long long grow0 = (long long)q0 * H + r0;  // global row of the tile's first row
  int row_local[2] = {rg * 16 + quad, rg * 16 + quad + 8};
  int pos_row[2], lo_row[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rr = r0 + row_local[i];
    pos_row[i] = rr < rows_b ? pos0 + rr / H : -1;  // -1: no key is visible to a row outside the sequence
    lo_row[i] = window > 0 ? pos_row[i] - window + 1 : 0;
  }

  const bool group_active = r0 + rg * 16 < rows_b;
  if (my_lo > my_hi) {  // nothing in this split's range: an empty partial
    if (splits > 1 && vq == 0 && qi == 0)
      for (int i = 0; i < 2; ++i)
        if (r0 + row_local[i] < rows_b) {
          part_m[(size_t)split * total_rows + grow0 + row_local[i]] = -INFINITY;
          part_l[(size_t)split * total_rows + grow0 + row_local[i]] = 0.f;
        }
    return;
  }

  const int* table = block_table + (size_t)b * max_blocks;
  // four threads copy one cached row (THREADS = 4 * BN): the page lookup is done once per row
  static_assert(THREADS == 4 * BN, "one cached row per four threads");
  auto load_keys = [&](int kb, int buf) {
    constexpr int CH = D / 8;
    const int key = threadIdx.x >> 2, sub = threadIdx.x & 3;
    const int j = kb * BN + key;
    __nv_bfloat16* d = Ks + ((size_t)buf * BN + key) * DS;
    if (j >= k_lo && j <= k_hi) {
      const __nv_bfloat16* src = cache + ((size_t)table[j / page] * page + (j % page)) * D;
#pragma unroll 6
      for (int part = sub; part < CH; part += 4) cp_async16(d + part * 8, src + part * 8);
    } else {
      for (int part = sub; part < CH; part += 4) *reinterpret_cast<uint4*>(d + part * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  {  // the query rows, with the first key block
    constexpr int CH = D / 8;
    for (int c = threadIdx.x; c < BM * CH; c += THREADS) {
      const int r = c / CH, part = c - r * CH;
      __nv_bfloat16* d = Qs + (size_t)r * DS + part * 8;
      if (r0 + r < rows_b)
        cp_async16(d, q_abs + (size_t)(grow0 + r) * D + part * 8);
      else
        *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  load_keys(my_lo, 0);
  cp_async_commit();

  float o[VT_W][4];
#pragma unroll
  for (int i = 0; i < VT_W; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int n_blocks = my_hi - my_lo + 1;
  for (int it = 0; it < n_blocks; ++it) {
    const int kb = my_lo + it, buf = it & 1;
    if (it + 1 < n_blocks) {
      load_keys(kb + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (group_active) {  // a row group without rows (a decode step of few heads) only helps with the copies
    const __nv_bfloat16* Kb = Ks + (size_t)buf * BN * DS;

    // S: this warp's 16 rows against its 16 keys.  Even and odd k-steps add into sums of their own, so
    // that four chains of dependent MMAs are in flight instead of two (a warp waits for an MMA's
    // result many cycles, and few warps are resident to fill them).
    float s[2][4] = {}, s_odd[2][4] = {};
#pragma unroll 2
    for (int ks = 0; ks < D / 16; ks += 2) {
      unsigned a[4], kf[4];
      ldmatrix_x4(a, Qs + (size_t)(rg * 16 + (lane & 15)) * DS + ks * 16 + (lane >> 4) * 8);
      ldmatrix_x4(kf, Kb + (size_t)(vq * 16 + (lane >> 4) * 8 + (lane & 7)) * DS + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], a, kf[0], kf[1]);
      mma_bf16(s[1], a, kf[2], kf[3]);
      if (ks + 1 < D / 16) {
        unsigned a2[4], kf2[4];
        ldmatrix_x4(a2, Qs + (size_t)(rg * 16 + (lane & 15)) * DS + (ks + 1) * 16 + (lane >> 4) * 8);
        ldmatrix_x4(kf2, Kb + (size_t)(vq * 16 + (lane >> 4) * 8 + (lane & 7)) * DS + (ks + 1) * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s_odd[0], a2, kf2[0], kf2[1]);
        mma_bf16(s_odd[1], a2, kf2[2], kf2[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] += s_odd[nt][e];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kb * BN + vq * 16 + nt * 8 + 2 * qi + (e & 1), r = e >> 1;
        if (key > pos_row[r] || key < lo_row[r]) s[nt][e] = -INFINITY;
        mx[r] = fmaxf(mx[r], s[nt][e]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      if (qi == 0) smax[(rg * 4 + vq) * 16 + quad + 8 * r] = mx[r];
    }
    group_barrier(rg);
    float m_use[2], corr[2], rsum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float m_new = m_run[r];
#pragma unroll
      for (int w = 0; w < 4; ++w) m_new = fmaxf(m_new, smax[(rg * 4 + w) * 16 + quad + 8 * r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f((m_run[r] - m_use[r]) * scale_log2);
      m_run[r] = m_new;
    }
    __nv_bfloat16* Pg = Ps + (size_t)rg * 16 * PS;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float p0 = exp2f((s[nt][2 * r] - m_use[r]) * scale_log2), p1 = exp2f((s[nt][2 * r + 1] - m_use[r]) * scale_log2);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        // the sum runs over the rounded weights, the ones the value product uses
        rsum[r] += __low2float(pb) + __high2float(pb);
        *reinterpret_cast<__nv_bfloat162*>(Pg + (size_t)(quad + 8 * r) * PS + vq * 16 + nt * 8 + 2 * qi) = pb;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rsum[r] += __shfl_xor_sync(0xffffffffu, rsum[r], 1);
      rsum[r] += __shfl_xor_sync(0xffffffffu, rsum[r], 2);
      if (qi == 0) ssum[(rg * 4 + vq) * 16 + quad + 8 * r] = rsum[r];
    }
    group_barrier(rg);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) t += ssum[(rg * 4 + w) * 16 + quad + 8 * r];
      l_run[r] = l_run[r] * corr[r] + t;
    }
#pragma unroll
    for (int i = 0; i < VT_W; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // O += P V: all 64 keys, this warp's value columns
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      unsigned a[4];
      ldmatrix_x4(a, Pg + (size_t)(lane & 15) * PS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int i = 0; i + 1 < VT_W; i += 2) {  // two value tiles per load where both exist
        const int tile = vq * VT_W + i;
        if (tile + 1 < VT) {
          unsigned vf[4];  // keys 0-7 / 8-15 of tile, then of tile + 1
          ldmatrix_x4_trans(vf, Kb + (size_t)(kk * 16 + (lane & 15)) * DS + tile * 8 + (lane >> 4) * 8);
          mma_bf16(o[i], a, vf[0], vf[1]);
          mma_bf16(o[i + 1], a, vf[2], vf[3]);
        } else if (tile < VT) {
          unsigned vf[2];
          ldmatrix_x2_trans(vf, Kb + (size_t)(kk * 16 + (lane & 15)) * DS + tile * 8);
          mma_bf16(o[i], a, vf[0], vf[1]);
        }
      }
      if (VT_W & 1) {
        const int tile = vq * VT_W + VT_W - 1;
        if (tile < VT) {
          unsigned vf[2];
          ldmatrix_x2_trans(vf, Kb + (size_t)(kk * 16 + (lane & 15)) * DS + tile * 8);
          mma_bf16(o[VT_W - 1], a, vf[0], vf[1]);
        }
      }
    }
    }
    __syncthreads();  // the buffer and P are written again in the next round
  }

  if (splits == 1) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r0 + row_local[r];
      if (rr >= rows_b) continue;
      const long long grow = grow0 + row_local[r];
      const float f = l_run[r] > 0.f ? (gates ? gates[grow] : 1.f) / l_run[r] : 0.f;
#pragma unroll
      for (int i = 0; i < VT_W; ++i) {
        const int tile = vq * VT_W + i;
        if (tile < VT)
          *reinterpret_cast<__nv_bfloat162*>(out + (size_t)grow * RANK + tile * 8 + 2 * qi) = __floats2bfloat162_rn(o[i][2 * r] * f, o[i][2 * r + 1] * f);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = r0 + row_local[r];
      if (rr >= rows_b) continue;
      const size_t prow = (size_t)split * total_rows + grow0 + row_local[r];
#pragma unroll
      for (int i = 0; i < VT_W; ++i) {
        const int tile = vq * VT_W + i;
        if (tile < VT) *reinterpret_cast<float2*>(part_o + prow * RANK + tile * 8 + 2 * qi) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
      }
      if (vq == 0 && qi == 0) {
        part_m[prow] = m_run[r];
        part_l[prow] = l_run[r];
      }
    }
  }
}

// Merges the splits of every row: weights exp2((m_s - max m) * scale), sums of the unnormalised
// rows and of their sums, one division, the gate.  The splits' maxima and sums are fetched by one
// thread each (all loads in flight at once) and turned into weights by the first warp; every
// thread then sums its columns with several loads in flight.
constexpr int MERGE_MAX_SPLITS = 64;

__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                                              const float* __restrict__ part_l, __nv_bfloat16* __restrict__ out,
                                              const float* __restrict__ gates, int splits, long long total_rows, float scale_log2) {
  ts_pdl_prologue();
  __shared__ float weight[MERGE_MAX_SPLITS];
  __shared__ float factor;
  const long long row = blockIdx.x;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (lane < splits) {
      m0 = part_m[(size_t)lane * total_rows + row];
      l0 = part_l[(size_t)lane * total_rows + row];
    }
    if (lane + 32 < splits) {
      m1 = part_m[(size_t)(lane + 32) * total_rows + row];
      l1 = part_l[(size_t)(lane + 32) * total_rows + row];
    }
    const float g = gates ? gates[row] : 1.f;
    const float m = ts_warp_max(fmaxf(m0, m1));
    const float w0 = (lane < splits && m0 != -INFINITY) ? exp2f((m0 - m) * scale_log2) : 0.f;
    const float w1 = (lane + 32 < splits && m1 != -INFINITY) ? exp2f((m1 - m) * scale_log2) : 0.f;
    const float l = ts_warp_sum(w0 * l0 + w1 * l1);
    weight[lane] = w0;
    weight[lane + 32] = w1;
    if (lane == 0) factor = l > 0.f ? g / l : 0.f;
  }
  __syncthreads();
  const float f = factor;
  for (int c = threadIdx.x; c < RANK; c += blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float w = weight[s];
      if (w != 0.f) acc += w * part_o[((size_t)s * total_rows + row) * RANK + c];  // an empty range left nothing to read
    }
    out[(size_t)row * RANK + c] = __float2bfloat16_rn(acc * f);
  }
}

}  // namespace

// Rows per CTA and keys per block, for whoever plans the splits.
TS_EXPORT int ts_latent_attention_mma_rows() { return BM; }
TS_EXPORT int ts_latent_attention_mma_keys() { return BN; }

// q_abs [T, H, rank+rot] bf16; cache [slots, rank+rot] bf16; out [T, H, rank] bf16; gates [T, H] f32 or null.
// scratch: splits * T * H * (rank + 2) floats when splits > 1.
TS_EXPORT int ts_latent_attention_mma(const void* q_abs, const void* cache, void* out, const float* gates, const int* cu_seqlens,
                                      const int* context_lens, const int* block_table, int max_blocks, int page, int num_seqs,
                                      int max_seqlen_q, int T, int H, float scale, int window, int splits, float* scratch, void* stream) {
  if (num_seqs <= 0 || T <= 0) return 0;
  if (H <= 0 || page <= 0 || max_blocks <= 0 || max_seqlen_q <= 0 || splits < 1 || (splits > 1 && !scratch)) return TS_ERR_BAD_ARGUMENT;
  if (SMEM_BYTES > 227 * 1024 || num_seqs > 65535 || splits > MERGE_MAX_SPLITS) return TS_ERR_UNSUPPORTED_SIZE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long long total_rows = (long long)T * H;
  float* part_o = scratch;
  float* part_m = scratch ? scratch + (size_t)splits * total_rows * RANK : nullptr;
  float* part_l = scratch ? part_m + (size_t)splits * total_rows : nullptr;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((unsigned)(((long long)max_seqlen_q * H + BM - 1) / BM), (unsigned)num_seqs, (unsigned)splits);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = ts_launch(latent_attention_mma_kernel, grid, dim3(THREADS), SMEM_BYTES, s, (const __nv_bfloat16*)q_abs, (const __nv_bfloat16*)cache,
                     (__nv_bfloat16*)out, gates, cu_seqlens, context_lens, block_table, max_blocks, page, H, scale_log2, window, splits,
                     part_o, part_m, part_l, total_rows);
  if (rc != 0 || splits == 1) return rc;
  return ts_launch(latent_attention_merge_kernel, dim3((unsigned)total_rows), dim3(RANK >= 256 ? 256 : 64), 0, s, (const float*)part_o,
                   (const float*)part_m, (const float*)part_l, (__nv_bfloat16*)out, gates, splits, total_rows, scale_log2);
}
