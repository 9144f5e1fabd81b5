// Grouped-query attention over a paged cache for heads of any size, with normed queries and keys, a query temperature
// that grows with the position, and a tanh soft cap on the scores (kernels.h: CapAttnGeom).  No rotation.
//
//   capattn_prep_kernel   per token: RMS norm of every query and key head (fp32), the query temperature, the cache write
//   capattn_mma_kernel    the same walk on the tensor cores for bf16 rows whose sizes fit the MMA tiles (see below)
//   capattn_mma_group_kernel   ... with the query heads of one key/value head in one CTA (2 to 8 heads per group)
//   capattn_kernel        (fp32 rows, any sizes; FMA pipe) one CTA per (tile of CAPATTN_TILE query tokens of one sequence, query head): the sequence's
//                         cache blocks are walked in ascending order from block 0, scores and the running softmax
//                         (maximum, sum, accumulators) are fp32, masked keys weigh exactly zero
//
// A query row's arithmetic depends on its own position and on the 32-token block grid of its sequence only: not on the
// tile it shares with other queries, on the other sequences of the step, or on which physical blocks hold the keys.
// The cache holds one row per token and layer: K [num_blocks][KV_BLOCK][kv_heads * dim], V [..][kv_heads * vdim], in the
// operand type (bf16 when serving, fp32 in the all-fp32 mode); the block ids are the engine's.
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

template <class T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// grid (T, ceil((heads + 2 kv_heads) / 4)), 128 threads: one warp per (token, query head | key head | value head)
constexpr int PREP_WARPS = 4;
template <class CT>
__global__ void __launch_bounds__(PREP_WARPS * 32)
capattn_prep_kernel(const float* __restrict__ y, int ldy, int q_off, int k_off, int v_off, CapAttnGeom g,
                    const float* __restrict__ w_q, const float* __restrict__ w_k, float eps,
                    const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, CT* __restrict__ q_out,
                    CT* __restrict__ k_cache, CT* __restrict__ v_cache) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, hh = blockIdx.y * PREP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (hh >= g.heads + 2 * g.kv_heads) return;
  const int slot = slot_mapping[t];
  if (hh < g.heads + g.kv_heads) {
    const bool is_q = hh < g.heads;
    const int h = is_q ? hh : hh - g.heads;
    const float* src = y + (size_t)t * ldy + (is_q ? q_off : k_off) + (size_t)h * g.dim;
    float ss = 0.f;
    for (int i = lane; i < g.dim; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum_f(ss);
    float rs = 1.f / sqrtf(ss / (float)g.dim + eps);
    const float* w = is_q ? w_q : w_k;
    if (is_q) {
      if (g.qt_every > 0) rs *= 1.f + g.qt_coef * logf((float)((positions[t] + 1) / g.qt_every) + 1.f);
      CT* dst = q_out + ((size_t)t * g.heads + h) * g.dim;
      for (int i = lane; i < g.dim; i += 32) stf(dst + i, src[i] * rs * w[i]);
    } else if (slot >= 0) {
      CT* dst = k_cache + ((size_t)slot * g.kv_heads + h) * g.dim;
      for (int i = lane; i < g.dim; i += 32) stf(dst + i, src[i] * rs * w[i]);
    }
  } else if (slot >= 0) {
    const int h = hh - g.heads - g.kv_heads;
    const float* src = y + (size_t)t * ldy + v_off + (size_t)h * g.vdim;
    CT* dst = v_cache + ((size_t)slot * g.kv_heads + h) * g.vdim;
    for (int i = lane; i < g.vdim; i += 32) stf(dst + i, src[i]);
  }
}

constexpr int CA_THREADS = 128, CA_QT = CAPATTN_TILE, CA_CC = CAPATTN_MAX_VDIM / CA_THREADS;
static_assert(CA_QT == 16 && CA_THREADS == 128, "score mapping: 4 warps x 4 queries x 32 keys");

template <class CT, class OT>
__global__ void __launch_bounds__(CA_THREADS)
capattn_kernel(const CT* __restrict__ q, const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
               const AttnSeq* __restrict__ seqs, const LatentTile* __restrict__ tiles,
               const int32_t* __restrict__ block_table, int bt_stride, const float* __restrict__ gate, int gate_ld,
               OT* __restrict__ out, CapAttnGeom g) {
  extern __shared__ __align__(16) float ca_smem[];
  const int d = g.dim, dv = g.vdim, ldk = d + 1;
  float* Qs = ca_smem;                        // [CA_QT][d]      scaled queries
  float* Ks = Qs + CA_QT * d;                 // [KV_BLOCK][d+1]
  float* Vs = Ks + KV_BLOCK * ldk;            // [KV_BLOCK][dv]
  float* Ps = Vs + KV_BLOCK * dv;             // [CA_QT][KV_BLOCK]
  float* alpha = Ps + CA_QT * KV_BLOCK;       // [CA_QT]
  float* lsum = alpha + CA_QT;                // [CA_QT]
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int h = blockIdx.y, kvh = h / (g.heads / g.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = sq.q_start + tl.q0;             // first query row of the tile in the flat batch
  const int pos0 = sq.kv_len - sq.q_len + tl.q0;   // its position
  const int nq = tl.nq;
  for (int i = tid; i < CA_QT * d; i += CA_THREADS) {
    const int qi = i / d, kk = i % d;
    Qs[i] = qi < nq ? ldf(q + ((size_t)(row0 + qi) * g.heads + h) * d + kk) * g.scale : 0.f;
  }
  float acc[CA_QT][CA_CC];
#pragma unroll
  for (int qi = 0; qi < CA_QT; ++qi)
#pragma unroll
    for (int cc = 0; cc < CA_CC; ++cc) acc[qi][cc] = 0.f;
  float m_run[4], l_run[4];   // this warp's four query rows (valid in every lane)
#pragma unroll
  for (int i = 0; i < 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }
  const int n_blocks = (pos0 + nq - 1) / KV_BLOCK + 1;   // blocks that hold a key some query of the tile sees
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  const float inv_cap = g.softcap > 0.f ? 1.f / g.softcap : 0.f;
  for (int b = 0; b < n_blocks; ++b) {
    const size_t blk = (size_t)bt[b];
    __syncthreads();   // the previous block's Ks / Vs / Ps are consumed (first pass: Qs complete)
    for (int i = tid; i < KV_BLOCK * d; i += CA_THREADS) {
      const int j = i / d, kk = i % d;
      Ks[j * ldk + kk] = ldf(k_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * d + kk);
    }
    for (int i = tid; i < KV_BLOCK * dv; i += CA_THREADS) {
      const int j = i / dv, cc = i % dv;
      Vs[i] = ldf(v_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * dv + cc);
    }
    __syncthreads();
    // ---- scores: lane = key, this warp's four queries
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * ldk;
    const float* qr = Qs + warp * 4 * d;
    for (int kk = 0; kk < d; ++kk) {
      const float kv = kr[kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(qr[i * d + kk], kv, s[i]);
    }
    const int kpos = b * KV_BLOCK + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = warp * 4 + i;
      const bool ok = qi < nq && kpos <= pos0 + qi;
      float sc = s[i];
      if (g.softcap > 0.f) sc = g.softcap * tanhf(sc * inv_cap);
      sc = ok ? sc : -INFINITY;
      const float m_new = fmaxf(m_run[i], warp_max_f(sc));
      const float p = ok ? expf(sc - m_new) : 0.f;
      const float al = m_new == -INFINITY ? 1.f : expf(m_run[i] - m_new);   // (-inf: nothing seen yet, nothing to scale)
      l_run[i] = fmaf(l_run[i], al, warp_sum_f(p));
      m_run[i] = m_new;
      Ps[qi * KV_BLOCK + lane] = p;
      if (lane == 0) alpha[qi] = al;
    }
    __syncthreads();
    // ---- weighted sum of the values: thread = value column(s), all queries of the tile
#pragma unroll
    for (int cc = 0; cc < CA_CC; ++cc) {
      const int c = tid + cc * CA_THREADS;
      if (c < dv) {
#pragma unroll
        for (int qi = 0; qi < CA_QT; ++qi)
          if (qi < nq) acc[qi][cc] *= alpha[qi];
        for (int j = 0; j < KV_BLOCK; ++j) {
          const float vv = Vs[j * dv + c];
#pragma unroll
          for (int qi = 0; qi < CA_QT; ++qi)
            if (qi < nq) acc[qi][cc] = fmaf(Ps[qi * KV_BLOCK + j], vv, acc[qi][cc]);
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) lsum[warp * 4 + i] = l_run[i];
  }
  __syncthreads();
#pragma unroll
  for (int cc = 0; cc < CA_CC; ++cc) {
    const int c = tid + cc * CA_THREADS;
    if (c < dv) {
#pragma unroll
      for (int qi = 0; qi < CA_QT; ++qi)
        if (qi < nq) {
          const size_t row = (size_t)(row0 + qi);
          float o = acc[qi][cc] / lsum[qi];
          if (gate != nullptr) o *= 1.f / (1.f + expf(-gate[row * gate_ld + (size_t)h * dv + c]));
          stf(out + (row * g.heads + h) * dv + c, o);
        }
    }
  }
}

// ---- tensor-core variant: bf16 queries and cache rows, dim a multiple of 16 (<= 16 MMA_KS), vdim a multiple of 8 (<= 32 MMA_NT
// per warp).  Both products on mma.sync m16n8k16 with fp32 accumulators: the tile's 16 queries are the M rows; for the scores
// each of the four warps owns 8 of a block's 32 keys (the query's A fragments stay in registers for the whole walk, the key
// rows are B fragments as they lie; the block after the current one lands in a second buffer through cp.async meanwhile), for the weighted sum each warp owns every fourth group of 8 value columns (value rows
// through ldmatrix.trans).  Scale, soft cap, mask and the running softmax are fp32 on the accumulator fragments; the
// weights are rounded to bf16 once and the SAME rounded numbers are summed for the normaliser.  Rows padded by 16 bytes keep
// every fragment load free of bank conflicts.  A row's arithmetic does not depend on the other rows of its tile.
constexpr int MMA_KS = 8, MMA_NT = 8;
__device__ __forceinline__ void ca_ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ca_ldsm_x2(uint32_t (&r)[2], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ca_ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ca_cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void ca_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(CA_THREADS)
capattn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, const AttnSeq* __restrict__ seqs,
                   const LatentTile* __restrict__ tiles, const int32_t* __restrict__ block_table, int bt_stride,
                   const float* __restrict__ gate, int gate_ld, __nv_bfloat16* __restrict__ out, CapAttnGeom g) {
  using bf = __nv_bfloat16;
  extern __shared__ __align__(16) uint8_t cam_smem[];
  const int d = g.dim, dv = g.vdim, LDK = d + 8, LDV = dv + 8, LDP = KV_BLOCK + 8;
  bf* Qs = reinterpret_cast<bf*>(cam_smem);            // [16][LDK]
  bf* Ks2 = Qs + CA_QT * LDK;                          // [2][32][LDK]   two blocks: one in use, the next one landing
  bf* Vs2 = Ks2 + 2 * KV_BLOCK * LDK;                  // [2][32][LDV]
  bf* Ps = Vs2 + 2 * KV_BLOCK * LDV;                   // [16][LDP]
  float* smax = reinterpret_cast<float*>(Ps + CA_QT * LDP);   // [4][16]; reused for the final row sums
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int h = blockIdx.y, kvh = h / (g.heads / g.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t2 = (lane & 3) * 2;
  const int row0 = sq.q_start + tl.q0, pos0 = sq.kv_len - sq.q_len + tl.q0, nq = tl.nq;
  const int dch = d / 8, vch = dv / 8;   // 16-byte chunks per row
  for (int i = tid; i < CA_QT * dch; i += CA_THREADS) {
    const int qi = i / dch, ch = i % dch;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qi < nq) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + qi) * g.heads + h) * d + ch * 8);
    *reinterpret_cast<uint4*>(Qs + qi * LDK + ch * 8) = v;
  }
  __syncthreads();
  const int nks = d / 16;
  uint32_t qa[MMA_KS][4];
#pragma unroll
  for (int ks = 0; ks < MMA_KS; ++ks)
    if (ks < nks) ca_ldsm_x4(qa[ks], Qs + (size_t)(lane & 15) * LDK + ks * 16 + (lane >> 4) * 8);
  float acc[MMA_NT][4];
#pragma unroll
  for (int j = 0; j < MMA_NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};   // rows gq and gq + 8
  const int n_blocks = (pos0 + nq - 1) / KV_BLOCK + 1;
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  const float inv_cap = g.softcap > 0.f ? 1.f / g.softcap : 0.f;
  // block b's K and V rows -> buffer b & 1, as 16-byte asynchronous copies (one commit group per block)
  auto fetch = [&](int b) {
    const size_t blk = (size_t)bt[b];
    bf* Kd = Ks2 + (size_t)(b & 1) * KV_BLOCK * LDK;
    bf* Vd = Vs2 + (size_t)(b & 1) * KV_BLOCK * LDV;
    for (int i = tid; i < KV_BLOCK * dch; i += CA_THREADS) {
      const int j = i / dch, ch = i % dch;
      ca_cp_async16(Kd + j * LDK + ch * 8, k_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * d + ch * 8);
    }
    for (int i = tid; i < KV_BLOCK * vch; i += CA_THREADS) {
      const int j = i / vch, ch = i % vch;
      ca_cp_async16(Vd + j * LDV + ch * 8, v_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * dv + ch * 8);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fetch(0);
  for (int b = 0; b < n_blocks; ++b) {
    // the other buffer was last read in the previous pass, which ended with a barrier
    if (b + 1 < n_blocks) {
      fetch(b + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();   // every thread's copies of block b have landed
    const bf* Ks = Ks2 + (size_t)(b & 1) * KV_BLOCK * LDK;
    const bf* Vs = Vs2 + (size_t)(b & 1) * KV_BLOCK * LDV;
    // ---- scores of this warp's 8 keys
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < MMA_KS; ++ks)
      if (ks < nks) {
        uint32_t kb[2];
        ca_ldsm_x2(kb, Ks + (size_t)(warp * 8 + (lane & 7)) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
        ca_mma(c, qa[ks], kb[0], kb[1]);
      }
    bool ok[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int qi = gq + (e >> 1) * 8, kpos = b * KV_BLOCK + warp * 8 + t2 + (e & 1);
      ok[e] = qi < nq && kpos <= pos0 + qi;
      float sc = c[e] * g.scale;
      if (g.softcap > 0.f) sc = g.softcap * tanhf(sc * inv_cap);
      c[e] = ok[e] ? sc : -INFINITY;
    }
    float mx[2] = {fmaxf(c[0], c[1]), fmaxf(c[2], c[3])};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if ((lane & 3) == 0) {
      smax[warp * CA_QT + gq] = mx[0];
      smax[warp * CA_QT + gq + 8] = mx[1];
    }
    __syncthreads();
    float al[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int qi = gq + r * 8;
      const float bm = fmaxf(fmaxf(smax[qi], smax[CA_QT + qi]), fmaxf(smax[2 * CA_QT + qi], smax[3 * CA_QT + qi]));
      const float m_new = fmaxf(m_run[r], bm);
      al[r] = m_new == -INFINITY ? 1.f : expf(m_run[r] - m_new);
      const bf p0 = __float2bfloat16_rn(ok[2 * r] ? expf(c[2 * r] - m_new) : 0.f);
      const bf p1 = __float2bfloat16_rn(ok[2 * r + 1] ? expf(c[2 * r + 1] - m_new) : 0.f);
      l_part[r] = fmaf(l_part[r], al[r], __bfloat162float(p0) + __bfloat162float(p1));
      m_run[r] = m_new;
      __nv_bfloat162 pk;
      pk.x = p0; pk.y = p1;
      *reinterpret_cast<__nv_bfloat162*>(Ps + qi * LDP + warp * 8 + t2) = pk;
    }
    __syncthreads();
    // ---- weighted sum of the values: this warp's groups of 8 columns
    uint32_t a0[4], a1[4];
    ca_ldsm_x4(a0, Ps + (size_t)(lane & 15) * LDP + (lane >> 4) * 8);
    ca_ldsm_x4(a1, Ps + (size_t)(lane & 15) * LDP + 16 + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n0 = (warp + 4 * j) * 8;
      if (n0 < dv) {
        acc[j][0] *= al[0]; acc[j][1] *= al[0]; acc[j][2] *= al[1]; acc[j][3] *= al[1];
        uint32_t vb[4];
        ca_ldsm_x4_trans(vb, Vs + (size_t)lane * LDV + n0);
        ca_mma(acc[j], a0, vb[0], vb[1]);
        ca_mma(acc[j], a1, vb[2], vb[3]);
      }
    }
    __syncthreads();   // this pass's buffers, maxima and weights are consumed
  }
  // ---- row sums: over the quad, then over the warps
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 1);
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 2);
  }
  __syncthreads();
  if ((lane & 3) == 0) {
    smax[warp * CA_QT + gq] = l_part[0];
    smax[warp * CA_QT + gq + 8] = l_part[1];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = gq + r * 8;
    if (qi >= nq) continue;
    const float inv_l = 1.f / (smax[qi] + smax[CA_QT + qi] + smax[2 * CA_QT + qi] + smax[3 * CA_QT + qi]);
    const size_t row = (size_t)(row0 + qi);
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n = (warp + 4 * j) * 8 + t2;
      if (n < dv) {
        float o0 = acc[j][2 * r] * inv_l, o1 = acc[j][2 * r + 1] * inv_l;
        if (gate != nullptr) {
          const float* gr = gate + row * gate_ld + (size_t)h * dv + n;
          o0 *= 1.f / (1.f + expf(-gr[0]));
          o1 *= 1.f / (1.f + expf(-gr[1]));
        }
        __nv_bfloat162 pk;
        pk.x = __float2bfloat16_rn(o0); pk.y = __float2bfloat16_rn(o1);
        *reinterpret_cast<__nv_bfloat162*>(out + (row * g.heads + h) * dv + n) = pk;
      }
    }
  }
}

// ---- grouped variant: the query heads that share a key/value head run in ONE CTA, one warp per head, so a block's K and V
// rows are fetched once per group.  A warp owns its head's whole 16 x 32 score tile: the running softmax needs no exchange
// between warps (row maxima and sums meet over the four lanes of a quad), the weights go from the score accumulators straight
// into the A fragments of the second product, and the only barriers are the two per block that guard the double buffer.
// vdim <= 8 MMG_NT.  Same arithmetic per row as capattn_mma_kernel.
constexpr int MMG_NT = 16;
__global__ void __launch_bounds__(256)
capattn_mma_group_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const AttnSeq* __restrict__ seqs,
                         const LatentTile* __restrict__ tiles, const int32_t* __restrict__ block_table, int bt_stride,
                         const float* __restrict__ gate, int gate_ld, __nv_bfloat16* __restrict__ out, CapAttnGeom g) {
  using bf = __nv_bfloat16;
  extern __shared__ __align__(16) uint8_t cag_smem[];
  const int d = g.dim, dv = g.vdim, LDK = d + 8, LDV = dv + 8;
  bf* Ks2 = reinterpret_cast<bf*>(cag_smem);           // [2][32][LDK]
  bf* Vs2 = Ks2 + 2 * KV_BLOCK * LDK;                  // [2][32][LDV]
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int gs = g.heads / g.kv_heads, kvh = blockIdx.y;
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t2 = (lane & 3) * 2;
  const int h = kvh * gs + warp;
  const int row0 = sq.q_start + tl.q0, pos0 = sq.kv_len - sq.q_len + tl.q0, nq = tl.nq;
  const int dch = d / 8, vch = dv / 8, nks = d / 16, nnt = dv / 8;
  uint32_t qa[MMA_KS][4];
#pragma unroll
  for (int ks = 0; ks < MMA_KS; ++ks) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int qi = gq + (e & 1) * 8, col = ks * 16 + t2 + (e >> 1) * 8;
      qa[ks][e] = (ks < nks && qi < nq) ? *reinterpret_cast<const uint32_t*>(q + ((size_t)(row0 + qi) * g.heads + h) * d + col) : 0u;
    }
  }
  float acc[MMG_NT][4];
#pragma unroll
  for (int j = 0; j < MMG_NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};
  const int n_blocks = (pos0 + nq - 1) / KV_BLOCK + 1;
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  const float inv_cap = g.softcap > 0.f ? 1.f / g.softcap : 0.f;
  auto fetch = [&](int b) {
    const size_t blk = (size_t)bt[b];
    bf* Kd = Ks2 + (size_t)(b & 1) * KV_BLOCK * LDK;
    bf* Vd = Vs2 + (size_t)(b & 1) * KV_BLOCK * LDV;
    for (int i = tid; i < KV_BLOCK * dch; i += nthr) {
      const int j = i / dch, ch = i % dch;
      ca_cp_async16(Kd + j * LDK + ch * 8, k_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * d + ch * 8);
    }
    for (int i = tid; i < KV_BLOCK * vch; i += nthr) {
      const int j = i / vch, ch = i % vch;
      ca_cp_async16(Vd + j * LDV + ch * 8, v_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * dv + ch * 8);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fetch(0);
  for (int b = 0; b < n_blocks; ++b) {
    if (b + 1 < n_blocks) {
      fetch(b + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();   // every thread's copies of block b have landed
    const bf* Ks = Ks2 + (size_t)(b & 1) * KV_BLOCK * LDK;
    const bf* Vs = Vs2 + (size_t)(b & 1) * KV_BLOCK * LDV;
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < MMA_KS; ++ks)
        if (ks < nks) {
          uint32_t kb[2];
          ca_ldsm_x2(kb, Ks + (size_t)(nt * 8 + (lane & 7)) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
          ca_mma(sc[nt], qa[ks], kb[0], kb[1]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qi = gq + (e >> 1) * 8, kpos = b * KV_BLOCK + nt * 8 + t2 + (e & 1);
        float v = sc[nt][e] * g.scale;
        if (g.softcap > 0.f) v = g.softcap * tanhf(v * inv_cap);
        v = (qi < nq && kpos <= pos0 + qi) ? v : -INFINITY;
        sc[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float al[2];
    uint32_t pa[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      al[r] = m_new == -INFINITY ? 1.f : expf(m_run[r] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float v0 = sc[nt][2 * r], v1 = sc[nt][2 * r + 1];
        __nv_bfloat162 pk;
        pk.x = __float2bfloat16_rn(v0 == -INFINITY ? 0.f : expf(v0 - m_new));
        pk.y = __float2bfloat16_rn(v1 == -INFINITY ? 0.f : expf(v1 - m_new));
        sum += __bfloat162float(pk.x) + __bfloat162float(pk.y);
        // keys nt * 8 + t2 (+1) of row gq + 8 r: A fragment of k-step nt / 2, register r (low key half) or r + 2 (high half)
        pa[nt >> 1][r + (nt & 1) * 2] = *reinterpret_cast<uint32_t*>(&pk);
      }
      l_part[r] = fmaf(l_part[r], al[r], sum);
      m_run[r] = m_new;
    }
#pragma unroll
    for (int j = 0; j < MMG_NT; ++j)
      if (j < nnt) {
        acc[j][0] *= al[0]; acc[j][1] *= al[0]; acc[j][2] *= al[1]; acc[j][3] *= al[1];
        uint32_t vb[4];
        ca_ldsm_x4_trans(vb, Vs + (size_t)lane * LDV + j * 8);
        ca_mma(acc[j], pa[0], vb[0], vb[1]);
        ca_mma(acc[j], pa[1], vb[2], vb[3]);
      }
    __syncthreads();   // this pass's buffer is consumed
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 1);
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 2);
    const int qi = gq + r * 8;
    if (qi >= nq) continue;
    const float inv_l = 1.f / l_part[r];
    const size_t row = (size_t)(row0 + qi);
#pragma unroll
    for (int j = 0; j < MMG_NT; ++j)
      if (j < nnt) {
        const int n = j * 8 + t2;
        float o0 = acc[j][2 * r] * inv_l, o1 = acc[j][2 * r + 1] * inv_l;
        if (gate != nullptr) {
          const float* gr = gate + row * gate_ld + (size_t)h * dv + n;
          o0 *= 1.f / (1.f + expf(-gr[0]));
          o1 *= 1.f / (1.f + expf(-gr[1]));
        }
        __nv_bfloat162 pk;
        pk.x = __float2bfloat16_rn(o0); pk.y = __float2bfloat16_rn(o1);
        *reinterpret_cast<__nv_bfloat162*>(out + (row * g.heads + h) * dv + n) = pk;
      }
  }
}

// TGIS_CAPATTN_GROUP=1 routes grouped-query shapes to capattn_mma_group_kernel (read at every launch).  Off by default: measured
// at 16 query / 4 key-value heads of 128 it is slower than one head per CTA (2048-token prefill step 172 against 148 us, a decode
// step of 32 sequences 0.87 against 0.76 ms per step for the whole model) -- a quarter of the CTAs, each warp walking its whole
// 16 x 32 tile alone with 162 registers, costs more than the K / V traffic it saves while the rows come out of L2.
bool capattn_group_on() {
  const char* e = getenv("TGIS_CAPATTN_GROUP");
  return e != nullptr && e[0] == '1';
}

bool capattn_mma_eligible(const CapAttnGeom& g, const void* q, const void* k_cache, const void* v_cache, const void* out) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TGIS_CAPATTN_MMA");   // 0: the FMA kernel for every shape (A/B and the tests)
    on = (e && e[0] == '0') ? 0 : 1;
  }
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return on == 1 && g.dim % 16 == 0 && g.dim <= 16 * MMA_KS && g.vdim % 8 == 0 && g.vdim <= 32 * MMA_NT && al16(q) &&
         al16(k_cache) && al16(v_cache) && al16(out);
}

size_t capattn_smem(const CapAttnGeom& g) {
  return ((size_t)CA_QT * g.dim + (size_t)KV_BLOCK * (g.dim + 1) + (size_t)KV_BLOCK * g.vdim + CA_QT * KV_BLOCK + 2 * CA_QT) *
         sizeof(float);
}

template <class CT, class OT>
cudaError_t capattn_launch_t(const void* q, const void* k_cache, const void* v_cache, const AttnSeq* seqs,
                             const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                             const float* gate, int gate_ld, void* out, const CapAttnGeom& g, cudaStream_t stream) {
  const size_t smem = capattn_smem(g);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    const cudaError_t e = cudaFuncSetAttribute(capattn_kernel<CT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    smem_set = smem;
  }
  return launch_k(capattn_kernel<CT, OT>, dim3(n_tiles, g.heads), dim3(CA_THREADS), smem, stream,
                  reinterpret_cast<const CT*>(q), reinterpret_cast<const CT*>(k_cache), reinterpret_cast<const CT*>(v_cache),
                  seqs, tiles, block_table, bt_stride, gate, gate_ld, reinterpret_cast<OT*>(out), g);
}

}  // namespace

cudaError_t capattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const CapAttnGeom& g,
                                const float* w_q, const float* w_k, float eps, const int32_t* positions,
                                const int32_t* slot_mapping, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  const dim3 grid(T, (g.heads + 2 * g.kv_heads + PREP_WARPS - 1) / PREP_WARPS);
  if (dtype == DT_BF16)
    return launch_k(capattn_prep_kernel<__nv_bfloat16>, grid, dim3(PREP_WARPS * 32), 0, stream, y, ldy, q_off, k_off, v_off, g, w_q, w_k,
                    eps, positions, slot_mapping, reinterpret_cast<__nv_bfloat16*>(q_out),
                    reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache));
  return launch_k(capattn_prep_kernel<float>, grid, dim3(PREP_WARPS * 32), 0, stream, y, ldy, q_off, k_off, v_off, g, w_q, w_k, eps,
                  positions, slot_mapping, reinterpret_cast<float*>(q_out), reinterpret_cast<float*>(k_cache),
                  reinterpret_cast<float*>(v_cache));
}

cudaError_t capattn_launch(const void* q, const void* k_cache, const void* v_cache, int dtype, const AttnSeq* seqs,
                           const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                           const float* gate, int gate_ld, void* out, int out_dtype, const CapAttnGeom& g,
                           cudaStream_t stream) {
  if (n_tiles <= 0) return cudaSuccess;
  if (g.heads < 1 || g.kv_heads < 1 || g.heads % g.kv_heads != 0 || g.heads > 65535 || g.dim < 1 || g.vdim < 1 ||
      g.vdim > CAPATTN_MAX_VDIM || capattn_smem(g) > 200 * 1024 || out_dtype != dtype)
    return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  if (dtype == DT_BF16 && capattn_mma_eligible(g, q, k_cache, v_cache, out) && g.heads / g.kv_heads >= 2 &&
      g.heads / g.kv_heads <= 8 && g.vdim <= 8 * MMG_NT && capattn_group_on()) {
    const size_t smem = ((size_t)2 * KV_BLOCK * (g.dim + 8) + (size_t)2 * KV_BLOCK * (g.vdim + 8)) * sizeof(bf);   // <= 35 KB
    return launch_k(capattn_mma_group_kernel, dim3(n_tiles, g.kv_heads), dim3(32 * (g.heads / g.kv_heads)), smem, stream,
                    reinterpret_cast<const bf*>(q), reinterpret_cast<const bf*>(k_cache), reinterpret_cast<const bf*>(v_cache), seqs,
                    tiles, block_table, bt_stride, gate, gate_ld, reinterpret_cast<bf*>(out), g);
  }
  if (dtype == DT_BF16 && capattn_mma_eligible(g, q, k_cache, v_cache, out)) {
    const size_t smem = ((size_t)(CA_QT + 2 * KV_BLOCK) * (g.dim + 8) + (size_t)2 * KV_BLOCK * (g.vdim + 8) + CA_QT * (KV_BLOCK + 8)) * sizeof(bf) +
                        4 * CA_QT * sizeof(float);   // <= 58 KB
    static bool attr_set = false;
    if (!attr_set) {
      const cudaError_t e = cudaFuncSetAttribute(capattn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    return launch_k(capattn_mma_kernel, dim3(n_tiles, g.heads), dim3(CA_THREADS), smem, stream, reinterpret_cast<const bf*>(q),
                    reinterpret_cast<const bf*>(k_cache), reinterpret_cast<const bf*>(v_cache), seqs, tiles, block_table, bt_stride,
                    gate, gate_ld, reinterpret_cast<bf*>(out), g);
  }
  if (dtype == DT_BF16)
    return capattn_launch_t<bf, bf>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, gate, gate_ld, out, g, stream);
  return capattn_launch_t<float, float>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, gate, gate_ld, out, g, stream);
}

}  // namespace tgis
