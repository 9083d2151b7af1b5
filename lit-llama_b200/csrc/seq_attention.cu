// Block-local causal softmax attention with a sink term, score soft-capping, grouped key/value heads, a per-head
// sigmoid output gate and a ring cache of one block of positions.
//
// A query at position p sees keys j <= p with j / block == p / block, so a sequence never needs more than `block`
// cached positions: entry p % block of the ring.  Keys of the portion being processed are read from the fresh
// projections (k_new / v_new), older ones of the same block from the ring; the ring is advanced AFTER the
// attention kernel (a second kernel in the same call), so a portion longer than a block cannot overwrite what it
// still has to read.
//
// attention kernel: WPQ warps per (query, head).  A warp takes batches of 32 consecutive keys: each lane scores one
// key (q from shared memory, its key row by 16-byte loads), the batch maximum and the weights go through shuffles,
// and the value rows are accumulated with lanes over value channels.  Scores, weights and accumulators are f32.
#include "seq_common.cuh"

namespace b2l {

constexpr int ATT_VMAX = 8;   // value channels per lane: V <= 256

template <typename act_t>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const act_t* __restrict__ k, int K, bool vec);

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int K, bool vec) {
  float s0 = 0.f, s1 = 0.f;
  if (vec) {
    for (int i = 0; i < K; i += 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(k + i);
      const float4 qa = *reinterpret_cast<const float4*>(q + i), qb = *reinterpret_cast<const float4*>(q + i + 4);
      s0 = fmaf(__uint_as_float(w.x << 16), qa.x, s0); s1 = fmaf(__uint_as_float(w.x & 0xffff0000u), qa.y, s1);
      s0 = fmaf(__uint_as_float(w.y << 16), qa.z, s0); s1 = fmaf(__uint_as_float(w.y & 0xffff0000u), qa.w, s1);
      s0 = fmaf(__uint_as_float(w.z << 16), qb.x, s0); s1 = fmaf(__uint_as_float(w.z & 0xffff0000u), qb.y, s1);
      s0 = fmaf(__uint_as_float(w.w << 16), qb.z, s0); s1 = fmaf(__uint_as_float(w.w & 0xffff0000u), qb.w, s1);
    }
  } else {
    for (int i = 0; i < K; ++i) s0 = fmaf(__bfloat162float(k[i]), q[i], s0);
  }
  return s0 + s1;
}

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int K, bool vec) {
  float s0 = 0.f, s1 = 0.f;
  if (vec) {
    for (int i = 0; i < K; i += 4) {
      const float4 w = *reinterpret_cast<const float4*>(k + i), qa = *reinterpret_cast<const float4*>(q + i);
      s0 = fmaf(w.x, qa.x, s0); s1 = fmaf(w.y, qa.y, s1);
      s0 = fmaf(w.z, qa.z, s0); s1 = fmaf(w.w, qa.w, s1);
    }
  } else {
    for (int i = 0; i < K; ++i) s0 = fmaf(k[i], q[i], s0);
  }
  return s0 + s1;
}

template <typename act_t, int WPQ>
__global__ void __launch_bounds__(128) seq_block_attention_kernel(b2l_seq_attn_args a, int vec) {
  extern __shared__ float smem[];
  constexpr int QPC = 4 / WPQ;                       // (query, head) pairs per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = a.K, V = a.V, Kpad = (K + 3) & ~3;
  float* sq = smem;                                  // [QPC][Kpad]
  float* sm = sq + QPC * Kpad;                       // merge area [4][2 + V]

  const int pair = blockIdx.x * QPC + warp / WPQ, sub = warp % WPQ;
  const bool live = pair < a.T * a.heads;
  const int t = live ? pair / a.heads : 0, h = live ? pair % a.heads : 0;
  const int g = h / (a.heads / a.kv_heads);
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int p = pos0 + t, c0 = (p / a.block) * a.block;       // first position of p's block

  float* myq = sq + (warp / WPQ) * Kpad;
  if (live && sub == 0)
    for (int i = lane; i < K; i += 32) myq[i] = a.q[((size_t)t * a.heads + h) * K + i];
  __syncthreads();

  const act_t* kn = (const act_t*)a.k_new;
  const act_t* vn = (const act_t*)a.v_new;
  const act_t* ck = (const act_t*)a.cache_k + (size_t)slot * a.block * a.kv_heads * K;
  const act_t* cv = (const act_t*)a.cache_v + (size_t)slot * a.block * a.kv_heads * V;

  float m = a.has_sink ? 0.f : -INFINITY, l = (a.has_sink && sub == 0) ? 1.f : 0.f;
  float acc[ATT_VMAX];
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) acc[c] = 0.f;

  if (live) {
    for (int jb = c0 + sub * 32; jb <= p; jb += 32 * WPQ) {
      const int j = jb + lane;
      float s = -INFINITY;
      if (j <= p) {
        const act_t* kr = j >= pos0 ? kn + ((size_t)(j - pos0) * a.kv_heads + g) * K
                                    : ck + ((size_t)(j - c0) * a.kv_heads + g) * K;
        s = dot_row<act_t>(myq, kr, K, vec != 0) * a.scale;
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
      }
      const float mn = fmaxf(m, warp_max(s));
      const float corr = expf(m - mn);                 // m = -inf only before the first batch without a sink: acc and l are 0
      const float w = j <= p ? expf(s - mn) : 0.f;
      l = l * (m == -INFINITY ? 0.f : corr) + warp_sum(w);
#pragma unroll
      for (int c = 0; c < ATT_VMAX; ++c) acc[c] *= (m == -INFINITY ? 0.f : corr);
      m = mn;
      const int nb = min(32, p - jb + 1);
      for (int jj = 0; jj < nb; ++jj) {
        const float wj = __shfl_sync(0xffffffffu, w, jj);
        const int jv = jb + jj;
        const act_t* vr = jv >= pos0 ? vn + (size_t)(jv - pos0) * a.ldv + (size_t)g * V
                                     : cv + ((size_t)(jv - c0) * a.kv_heads + g) * V;
#pragma unroll
        for (int c = 0; c < ATT_VMAX; ++c) {
          const int ch = c * 32 + lane;
          if (ch < V) acc[c] = fmaf(wj, ld_act(vr, ch), acc[c]);
        }
      }
    }
  }

  if (WPQ > 1) {   // merge the partial softmaxes of the WPQ warps of this pair (QPC == 1)
    float* mine = sm + warp * (2 + ATT_VMAX * 32);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int c = 0; c < ATT_VMAX; ++c) mine[2 + c * 32 + lane] = acc[c];
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < WPQ; ++w) M = fmaxf(M, sm[w * (2 + ATT_VMAX * 32)]);
    l = 0.f;
#pragma unroll
    for (int c = 0; c < ATT_VMAX; ++c) acc[c] = 0.f;
    for (int w = 0; w < WPQ; ++w) {
      const float* o = sm + w * (2 + ATT_VMAX * 32);
      const float f = o[0] == -INFINITY ? 0.f : expf(o[0] - M);
      l += o[1] * f;
#pragma unroll
      for (int c = 0; c < ATT_VMAX; ++c) acc[c] += o[2 + c * 32 + lane] * f;
    }
  }
  if (!live) return;
  float f = a.out_mult / l;
  if (a.gate) f *= sigmoid_f(ld_act((const act_t*)a.gate, (size_t)t * a.ldg + h));
  act_t* o = (act_t*)a.out + (size_t)t * a.ldo + (size_t)h * V;
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) {
    const int ch = c * 32 + lane;
    if (ch < V) st_act(o, ch, acc[c] * f);
  }
}

// ring[p % block] <- token p for the portion's tokens in the block of its last token.
template <typename act_t>
__global__ void seq_ring_append_kernel(b2l_seq_attn_args a) {
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int last = pos0 + a.T - 1, c0 = (last / a.block) * a.block;
  const int first = max(pos0, c0);
  const int p = first + blockIdx.x;
  if (p > last) return;
  const int t = p - pos0, e = p - c0;
  const int nk = a.kv_heads * a.K, nv = a.kv_heads * a.V;
  const act_t* kn = (const act_t*)a.k_new + (size_t)t * nk;
  const act_t* vn = (const act_t*)a.v_new + (size_t)t * a.ldv;
  act_t* ck = (act_t*)a.cache_k + ((size_t)slot * a.block + e) * nk;
  act_t* cv = (act_t*)a.cache_v + ((size_t)slot * a.block + e) * nv;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) ck[i] = kn[i];
  for (int i = threadIdx.x; i < nv; i += blockDim.x) cv[i] = vn[i];
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_block_attention(const b2l_seq_attn_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_block_attention: null argument block");
  B2L_CHECK_ARG(a->q && a->k_new && a->v_new && a->cache_k && a->cache_v && a->meta && a->out, "b2l_seq_block_attention: null pointer");
  B2L_CHECK_ARG(a->T >= 0 && a->heads > 0 && a->kv_heads > 0 && a->K > 0 && a->V > 0 && a->block > 0, "b2l_seq_block_attention: bad size");
  B2L_CHECK_ARG(a->heads % a->kv_heads == 0, "b2l_seq_block_attention: heads %d not a multiple of kv_heads %d", a->heads, a->kv_heads);
  B2L_CHECK_SUPPORTED(a->V <= ATT_VMAX * 32, "b2l_seq_block_attention: value size %d above %d", a->V, ATT_VMAX * 32);
  B2L_CHECK_ARG(a->act_dtype == B2L_BF16 || a->act_dtype == B2L_F32, "b2l_seq_block_attention: act_dtype %d unsupported", a->act_dtype);
  if (a->T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t esz = a->act_dtype == B2L_BF16 ? 2 : 4;
  const int vec = ((a->K * esz) % 16 == 0) && (((uintptr_t)a->k_new | (uintptr_t)a->cache_k) % 16 == 0) && (a->K % 8 == 0 || esz == 4);
  const int pairs = a->T * a->heads;
  const int Kpad = (a->K + 3) & ~3;
  const bool split = pairs < 2 * sm_count();          // few queries (decoding): four warps share one query's keys
  const size_t smem = sizeof(float) * ((size_t)(split ? 1 : 4) * Kpad + 4 * (2 + ATT_VMAX * 32));
  B2L_CHECK_SUPPORTED(smem <= 48 * 1024, "b2l_seq_block_attention: key size %d too large", a->K);
  if (a->act_dtype == B2L_BF16) {
    if (split) seq_block_attention_kernel<__nv_bfloat16, 4><<<pairs, 128, smem, s>>>(*a, vec);
    else seq_block_attention_kernel<__nv_bfloat16, 1><<<(pairs + 3) / 4, 128, smem, s>>>(*a, vec);
  } else {
    if (split) seq_block_attention_kernel<float, 4><<<pairs, 128, smem, s>>>(*a, vec);
    else seq_block_attention_kernel<float, 1><<<(pairs + 3) / 4, 128, smem, s>>>(*a, vec);
  }
  B2L_LAUNCH_CHECK("seq_block_attention_kernel");
  const int n_app = std::min(a->T, a->block);
  if (a->act_dtype == B2L_BF16) seq_ring_append_kernel<__nv_bfloat16><<<n_app, 128, 0, s>>>(*a);
  else seq_ring_append_kernel<float><<<n_app, 128, 0, s>>>(*a);
  B2L_LAUNCH_CHECK("seq_ring_append_kernel");
  return 0;
}
