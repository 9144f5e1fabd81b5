// Grouped-query attention over a paged cache for heads of any size, with normed queries and keys, a query temperature
// that grows with the position, and a tanh soft cap on the scores (kernels.h: CapAttnGeom).  No rotation.
//
//   capattn_prep_kernel   per token: RMS norm of every query and key head (fp32), the query temperature, the cache write
//   capattn_kernel        one CTA per (tile of CAPATTN_TILE query tokens of one sequence, query head): the sequence's
//                         cache blocks are walked in ascending order from block 0, scores and the running softmax
//                         (maximum, sum, accumulators) are fp32, masked keys weigh exactly zero
//
// A query row's arithmetic depends on its own position and on the 32-token block grid of its sequence only: not on the
// tile it shares with other queries, on the other sequences of the step, or on which physical blocks hold the keys.
// The cache holds one row per token and layer: K [num_blocks][KV_BLOCK][kv_heads * dim], V [..][kv_heads * vdim], in the
// operand type (bf16 when serving, fp32 in the all-fp32 mode); the block ids are the engine's.
#include <cmath>
#include <cstdint>

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

// grid (T, heads + kv_heads): one warp-sized CTA per (token, query or key head); block z = 1 copies the values
template <class CT>
__global__ void __launch_bounds__(32)
capattn_prep_kernel(const float* __restrict__ y, int ldy, int q_off, int k_off, int v_off, CapAttnGeom g,
                    const float* __restrict__ w_q, const float* __restrict__ w_k, float eps,
                    const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, CT* __restrict__ q_out,
                    CT* __restrict__ k_cache, CT* __restrict__ v_cache) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, hh = blockIdx.y, lane = threadIdx.x;
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
  const dim3 grid(T, g.heads + 2 * g.kv_heads);
  if (dtype == DT_BF16)
    return launch_k(capattn_prep_kernel<__nv_bfloat16>, grid, dim3(32), 0, stream, y, ldy, q_off, k_off, v_off, g, w_q, w_k,
                    eps, positions, slot_mapping, reinterpret_cast<__nv_bfloat16*>(q_out),
                    reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache));
  return launch_k(capattn_prep_kernel<float>, grid, dim3(32), 0, stream, y, ldy, q_off, k_off, v_off, g, w_q, w_k, eps,
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
  if (dtype == DT_BF16)
    return capattn_launch_t<bf, bf>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, gate, gate_ld, out, g, stream);
  return capattn_launch_t<float, float>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, gate, gate_ld, out, g, stream);
}

}  // namespace tgis
