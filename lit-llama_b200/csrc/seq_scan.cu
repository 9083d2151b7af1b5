// Linear recurrences with a matrix state per head (gated delta rule, gated linear attention, state-space duality)
// as ONE kernel: S <- diag(d) S; [u = sigmoid(beta)(v - S^T k)]; S <- S + k u^T; o = S^T q.
//
// A CTA owns one head and a tile of value columns; a column of S (K numbers) lives in the registers of R adjacent
// lanes (SCAN_KPT numbers each), so a step is R-lane shuffles and no shared-memory traffic for S.  The state is
// read once, carried through all T tokens of the portion and written once ([V][K] per head, K fastest, so the R
// lanes of a column read consecutive 16-byte words).  Inputs of SCAN_TC steps are staged in shared memory by the
// whole CTA with asynchronous copies, one stage ahead of the recurrence.  All arithmetic is f32.
#include "seq_common.cuh"

namespace b2l {

constexpr int SCAN_KPT = 16;       // state numbers per lane
constexpr int SCAN_TC = 16;        // steps per shared-memory stage
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Inputs of SCAN_TC steps go to shared memory with cp.async, two stages deep: stage s+1 is in flight while the
// recurrence runs over stage s, so the sequential loop never waits on global memory after the first stage.
// Stage layout: q[TC][KP] k[TC][KP] d[TC][DP] v[TC][cols] vs[TC] beta[TC] (+ 2*TC unused: stages stay 16-byte aligned).
// PASS 0: the recurrence with outputs, from the slot's state (one chunk) or from a chunk's start state in the workspace.
// PASS 1: a chunk's local end state from zero and its total decay, no outputs (first pass of a chunked portion).
// CPL: value columns per lane.  A step reads k, q and d from shared memory once per lane, so with one column the loop is
// bound by shared-memory bandwidth (12 16-byte reads for 48 FMAs); two columns halve that where throughput matters (long
// portions without the delta rule); one column keeps the most CTAs for single tokens and the latency-bound delta rule.
template <int DELTA, typename act_t, int PASS, int CPL>
__global__ void __launch_bounds__(SCAN_THREADS, DELTA ? 2 : 3) seq_scan_kernel(b2l_seq_scan_args a, int R, int vec, int chunk_len) {
  extern __shared__ __align__(16) float smem[];
  const int KP = R * SCAN_KPT;                 // padded key size
  const int ncg = SCAN_THREADS / R;            // column groups: lane cidx holds columns cidx + j * ncg
  const int cols = ncg * CPL;                  // value columns of this CTA
  const int DP = a.decay_per_channel ? KP : 4;
  const int stage = SCAN_TC * (2 * KP + DP + cols + 4);
  const int beta_at = SCAN_TC * (2 * KP + DP + cols + 1);
  float* so = smem + 2 * stage;                // [TC][cols]

  const int tid = threadIdx.x, r = tid % R, cidx = tid / R;
  const int h = blockIdx.y, hq = h / (a.heads / a.qk_heads);
  const int v0 = blockIdx.x * cols;
  const int K = a.K, V = a.V;
  const int slot = a.meta[0];
  const bool chunked = a.n_chunks > 1;
  const int t_begin = blockIdx.z * chunk_len, t_end = min(a.T, t_begin + chunk_len);
  float* st = chunked ? a.work_state + ((size_t)blockIdx.z * a.heads + h) * (size_t)V * K
                      : a.state + ((size_t)slot * a.heads + h) * (size_t)V * K;
  const float skip = a.skip ? ld_act((const act_t*)a.skip, h) : 0.f;
  const float* gq = a.q + (size_t)hq * K;
  const float* gk = a.k + (size_t)hq * K;
  const float* gv = a.v + (size_t)h * V + v0;
  const float* gd = a.decay + (a.decay_per_channel ? (size_t)h * K : (size_t)h);
  const int ncol = min(cols, V - v0);

  // padding that no copy ever touches: q = k = 0 and d = 1 beyond K, v = 0 beyond V, vs = 1 without a value scale
  for (int b = 0; b < 2; ++b) {
    float* sq = smem + b * stage;
    float* sk = sq + SCAN_TC * KP;
    float* sd = sk + SCAN_TC * KP;
    float* sv = sd + SCAN_TC * DP;
    float* svs = sv + SCAN_TC * cols;
    for (int i = tid; i < SCAN_TC * KP; i += SCAN_THREADS) {
      if (i % KP >= K) {
        sq[i] = 0.f;
        sk[i] = 0.f;
        if (a.decay_per_channel) sd[i] = 1.f;
      }
    }
    for (int i = tid; i < SCAN_TC * cols; i += SCAN_THREADS)
      if (i % cols >= ncol) sv[i] = 0.f;
    if (tid < SCAN_TC) svs[tid] = 1.f;
  }

  auto prefetch = [&](int t0, int b) {
    const int nt = min(SCAN_TC, t_end - t0);
    float* sq = smem + b * stage;
    float* sk = sq + SCAN_TC * KP;
    float* sd = sk + SCAN_TC * KP;
    float* sv = sd + SCAN_TC * DP;
    float* svs = sv + SCAN_TC * cols;
    if (vec) {
      const int K4 = K >> 2;
      for (int i = tid; i < nt * K4; i += SCAN_THREADS) {
        const int t = i / K4, kk = (i - t * K4) << 2;
        cp_async16(sq + t * KP + kk, gq + (size_t)(t0 + t) * a.ldq + kk);
        cp_async16(sk + t * KP + kk, gk + (size_t)(t0 + t) * a.ldk + kk);
        if (a.decay_per_channel) cp_async16(sd + t * KP + kk, gd + (size_t)(t0 + t) * a.ldd + kk);
      }
    } else {
      for (int i = tid; i < nt * K; i += SCAN_THREADS) {
        const int t = i / K, kk = i - t * K;
        cp_async4(sq + t * KP + kk, gq + (size_t)(t0 + t) * a.ldq + kk);
        cp_async4(sk + t * KP + kk, gk + (size_t)(t0 + t) * a.ldk + kk);
        if (a.decay_per_channel) cp_async4(sd + t * KP + kk, gd + (size_t)(t0 + t) * a.ldd + kk);
      }
    }
    for (int i = tid; i < nt * ncol; i += SCAN_THREADS) {
      const int t = i / ncol, c = i - t * ncol;
      cp_async4(sv + t * cols + c, gv + (size_t)(t0 + t) * a.ldv + c);
    }
    if (tid < nt) {
      if (!a.decay_per_channel) cp_async4(sd + tid, gd + (size_t)(t0 + tid) * a.ldd);
      if (a.vscale) cp_async4(svs + tid, a.vscale + (size_t)(t0 + tid) * a.ldvs + h);
    }
    cp_async_commit();
  };
  auto beta_of = [&](int t0) -> float {   // raw gate of step t0 + tid: act-typed, so a plain load kept in a register
    return (DELTA && tid < min(SCAN_TC, t_end - t0)) ? ld_act((const act_t*)a.beta, (size_t)(t0 + tid) * a.ldb + h) : 0.f;
  };

  float S[CPL][SCAN_KPT];
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    const int vcol = v0 + cidx + j * ncg;
#pragma unroll
    for (int i = 0; i < SCAN_KPT; ++i) {
      const int kk = ((i >> 2) * R + r) * 4 + (i & 3);
      S[j][i] = (PASS == 0 && kk < K && vcol < V) ? st[(size_t)vcol * K + kk] : 0.f;
    }
  }
  float P[PASS ? SCAN_KPT : 1];       // PASS 1: the chunk's total decay of this lane's key channels
#pragma unroll
  for (int i = 0; i < (PASS ? SCAN_KPT : 1); ++i) P[i] = 1.f;

  __syncthreads();                    // the padding is written before any copy lands next to it
  prefetch(t_begin, 0);
  if (DELTA && tid < SCAN_TC) smem[beta_at + tid] = sigmoid_f(beta_of(t_begin));

  int b = 0;
  for (int t0 = t_begin; t0 < t_end; t0 += SCAN_TC, b ^= 1) {
    const int nt = min(SCAN_TC, t_end - t0);
    const bool more = t0 + SCAN_TC < t_end;
    float beta_next = 0.f;
    if (more) {
      prefetch(t0 + SCAN_TC, b ^ 1);
      beta_next = beta_of(t0 + SCAN_TC);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                  // stage t0 has landed for every thread; so[] of the previous stage is written out
    const float* sq = smem + b * stage;
    const float* sk = sq + SCAN_TC * KP;
    const float* sd = sk + SCAN_TC * KP;
    const float* sv = sd + SCAN_TC * DP;
    const float* svs = sv + SCAN_TC * cols;
    const float* sb = svs + SCAN_TC;

#pragma unroll(DELTA ? 2 : 1)
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * KP);
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * KP);
      float kr[SCAN_KPT], qr[SCAN_KPT];
#pragma unroll
      for (int i4 = 0; i4 < SCAN_KPT / 4; ++i4) {
        const float4 kv = k4[i4 * R + r], qv = q4[i4 * R + r];
        kr[i4 * 4 + 0] = kv.x; kr[i4 * 4 + 1] = kv.y; kr[i4 * 4 + 2] = kv.z; kr[i4 * 4 + 3] = kv.w;
        qr[i4 * 4 + 0] = qv.x; qr[i4 * 4 + 1] = qv.y; qr[i4 * 4 + 2] = qv.z; qr[i4 * 4 + 3] = qv.w;
      }
      if (a.decay_per_channel) {
        const float4* d4 = reinterpret_cast<const float4*>(sd + t * KP);
#pragma unroll
        for (int i4 = 0; i4 < SCAN_KPT / 4; ++i4) {
          const float4 dv = d4[i4 * R + r];
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            S[j][i4 * 4 + 0] *= dv.x; S[j][i4 * 4 + 1] *= dv.y; S[j][i4 * 4 + 2] *= dv.z; S[j][i4 * 4 + 3] *= dv.w;
          }
          if (PASS) { P[i4 * 4 + 0] *= dv.x; P[i4 * 4 + 1] *= dv.y; P[i4 * 4 + 2] *= dv.z; P[i4 * 4 + 3] *= dv.w; }
        }
      } else {
        const float d = sd[t];
#pragma unroll
        for (int j = 0; j < CPL; ++j)
#pragma unroll
          for (int i = 0; i < SCAN_KPT; ++i) S[j][i] *= d;
        if (PASS) P[0] *= d;
      }
      float vraw[CPL], u[CPL], o[CPL];
#pragma unroll
      for (int j = 0; j < CPL; ++j) {
        vraw[j] = sv[t * cols + cidx + j * ncg];
        u[j] = vraw[j] * svs[t];
      }
      if (PASS) {
#pragma unroll
        for (int j = 0; j < CPL; ++j)
#pragma unroll
          for (int i = 0; i < SCAN_KPT; ++i) S[j][i] = fmaf(kr[i], u[j], S[j][i]);
        continue;
      }
      if (DELTA) {
        // With S' = diag(d) S:  u = beta (v - S'^T k)  and  o = (S' + k u^T)^T q = S'^T q + u (k.q): the dot products
        // over this lane's channels are reduced together, so a step has ONE shuffle chain on its critical path.
        float c0 = 0.f, c1 = 0.f;
#pragma unroll
        for (int i = 0; i < SCAN_KPT; i += 2) {
          c0 = fmaf(kr[i], qr[i], c0);
          c1 = fmaf(kr[i + 1], qr[i + 1], c1);
        }
        float kq = c0 + c1, p[CPL], oq[CPL];
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          float p0 = 0.f, p1 = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
          for (int i = 0; i < SCAN_KPT; i += 2) {
            p0 = fmaf(S[j][i], kr[i], p0); p1 = fmaf(S[j][i + 1], kr[i + 1], p1);
            o0 = fmaf(S[j][i], qr[i], o0); o1 = fmaf(S[j][i + 1], qr[i + 1], o1);
          }
          p[j] = p0 + p1;
          oq[j] = o0 + o1;
        }
        for (int w = 1; w < R; w <<= 1) {
          kq += __shfl_xor_sync(0xffffffffu, kq, w);
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            p[j] += __shfl_xor_sync(0xffffffffu, p[j], w);
            oq[j] += __shfl_xor_sync(0xffffffffu, oq[j], w);
          }
        }
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          u[j] = sb[t] * (u[j] - p[j]);
#pragma unroll
          for (int i = 0; i < SCAN_KPT; ++i) S[j][i] = fmaf(kr[i], u[j], S[j][i]);
          o[j] = fmaf(u[j], kq, oq[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
          for (int i = 0; i < SCAN_KPT; i += 4) {
            S[j][i] = fmaf(kr[i], u[j], S[j][i]); S[j][i + 1] = fmaf(kr[i + 1], u[j], S[j][i + 1]);
            S[j][i + 2] = fmaf(kr[i + 2], u[j], S[j][i + 2]); S[j][i + 3] = fmaf(kr[i + 3], u[j], S[j][i + 3]);
            o0 = fmaf(S[j][i], qr[i], o0); o1 = fmaf(S[j][i + 1], qr[i + 1], o1);
            o2 = fmaf(S[j][i + 2], qr[i + 2], o2); o3 = fmaf(S[j][i + 3], qr[i + 3], o3);
          }
          o[j] = (o0 + o1) + (o2 + o3);
        }
        for (int w = 1; w < R; w <<= 1) {
#pragma unroll
          for (int j = 0; j < CPL; ++j) o[j] += __shfl_xor_sync(0xffffffffu, o[j], w);
        }
      }
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < CPL; ++j) so[t * cols + cidx + j * ncg] = o[j] * a.q_mult + skip * vraw[j];
      }
    }
    __syncthreads();
    if (PASS == 0) {
      for (int i = tid; i < nt * ncol; i += SCAN_THREADS) {
        const int t = i / ncol, c = i - t * ncol;
        a.out[(size_t)(t0 + t) * a.ldo + (size_t)h * V + v0 + c] = so[t * cols + c];
      }
    }
    if (DELTA && more && tid < SCAN_TC) smem[(b ^ 1) * stage + beta_at + tid] = sigmoid_f(beta_next);
  }

  if (PASS == 0 && chunked) return;   // chunk outputs: the slot's state is written by the combine kernel
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    const int vcol = v0 + cidx + j * ncg;
#pragma unroll
    for (int i = 0; i < SCAN_KPT; ++i) {
      const int kk = ((i >> 2) * R + r) * 4 + (i & 3);
      if (kk < K && vcol < V) st[(size_t)vcol * K + kk] = S[j][i];
    }
  }
  if (PASS && blockIdx.x == 0 && cidx == 0) {
    float* wd = a.work_decay + ((size_t)blockIdx.z * a.heads + h) * (a.decay_per_channel ? K : 1);
    if (a.decay_per_channel) {
#pragma unroll
      for (int i = 0; i < SCAN_KPT; ++i) {
        const int kk = ((i >> 2) * R + r) * 4 + (i & 3);
        if (kk < K) wd[kk] = P[i];
      }
    } else if (r == 0) {
      wd[0] = P[0];
    }
  }
}

// Between the passes of a chunked portion: work_state[c] (a chunk's local end state) becomes the chunk's START state,
// s_0 = the slot's state, s_(c+1) = D_c s_c + local_c, and the slot's state becomes s_n.  One thread per state entry.
__global__ void seq_scan_combine_kernel(b2l_seq_scan_args a) {
  const size_t per_head = (size_t)a.V * a.K, n = (size_t)a.heads * per_head;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int h = (int)(i / per_head), kk = (int)(i % a.K);
  float* st = a.state + (size_t)a.meta[0] * n;
  float s = st[i];
  const size_t dstep = (size_t)a.heads * (a.decay_per_channel ? a.K : 1);
  const float* dp = a.work_decay + (size_t)h * (a.decay_per_channel ? a.K : 1) + (a.decay_per_channel ? kk : 0);
  for (int c0 = 0; c0 < a.n_chunks; c0 += 8) {        // eight chunks' operands are requested together
    float d[8], local[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool in = c0 + u < a.n_chunks;
      d[u] = in ? dp[(size_t)(c0 + u) * dstep] : 1.f;
      local[u] = in ? a.work_state[(size_t)(c0 + u) * n + i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + u < a.n_chunks) a.work_state[(size_t)(c0 + u) * n + i] = s;
      s = fmaf(d[u], s, local[u]);
    }
  }
  st[i] = s;
}

static DynSmemCache g_scan_smem[10];
constexpr int SCAN_CHUNK = 128;      // tokens per chunk of a chunked portion (a multiple of SCAN_TC)

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_scan_chunks(int T, int delta) {
  if (delta || T < 2 * SCAN_CHUNK) return 1;
  return (T + SCAN_CHUNK - 1) / SCAN_CHUNK;
}

extern "C" int b2l_seq_scan(const b2l_seq_scan_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_scan: null argument block");
  B2L_CHECK_ARG(a->q && a->k && a->v && a->decay && a->state && a->meta && a->out, "b2l_seq_scan: null pointer");
  B2L_CHECK_ARG(!a->delta || a->beta, "b2l_seq_scan: the delta rule needs beta");
  B2L_CHECK_ARG(a->T >= 0 && a->heads > 0 && a->qk_heads > 0 && a->K > 0 && a->V > 0, "b2l_seq_scan: bad size");
  B2L_CHECK_ARG(a->heads % a->qk_heads == 0, "b2l_seq_scan: heads %d not a multiple of qk_heads %d", a->heads, a->qk_heads);
  B2L_CHECK_SUPPORTED(a->K <= 32 * SCAN_KPT, "b2l_seq_scan: key size %d above %d", a->K, 32 * SCAN_KPT);
  B2L_CHECK_ARG(a->n_chunks <= 1 || (!a->delta && a->work_state && a->work_decay && a->n_chunks == (a->T + SCAN_CHUNK - 1) / SCAN_CHUNK),
                "b2l_seq_scan: chunked portions need the workspace, no delta rule and n_chunks from b2l_seq_scan_chunks");
  if (a->T == 0) return 0;
  const int n_chunks = a->n_chunks > 1 ? a->n_chunks : 1;
  const int chunk_len = n_chunks > 1 ? SCAN_CHUNK : a->T;
  int R = 1;
  while (R * SCAN_KPT < a->K) R <<= 1;
  // two columns per lane where the loop is bound by shared-memory reads: long portions without the delta rule
  const int cpl = (!a->delta && a->T >= 64 && a->V >= 2 * (SCAN_THREADS / R)) ? 2 : 1;
  const int KP = R * SCAN_KPT, cols = (SCAN_THREADS / R) * cpl;
  const size_t smem = sizeof(float) * (2 * (size_t)SCAN_TC * (2 * KP + (a->decay_per_channel ? KP : 4) + cols + 4) + (size_t)SCAN_TC * cols);
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const int vec = a->K % 4 == 0 && a->ldq % 4 == 0 && a->ldk % 4 == 0 && al16(a->q) && al16(a->k) &&
                  (!a->decay_per_channel || (a->ldd % 4 == 0 && al16(a->decay)));
  dim3 grid((unsigned)((a->V + cols - 1) / cols), (unsigned)a->heads, (unsigned)n_chunks);
  cudaStream_t s = (cudaStream_t)stream;
#define B2L_SCAN_LAUNCH(D, T_, P_, C_, slot_)                                                 \
  do {                                                                                        \
    int rc_ = ensure_dyn_smem(seq_scan_kernel<D, T_, P_, C_>, smem, g_scan_smem[slot_]);      \
    if (rc_) return rc_;                                                                      \
    seq_scan_kernel<D, T_, P_, C_><<<grid, SCAN_THREADS, smem, s>>>(*a, R, vec, chunk_len);   \
  } while (0)
  const bool bf = a->act_dtype == B2L_BF16;
  if (!bf && a->act_dtype != B2L_F32) {
    set_error("b2l_seq_scan: act_dtype %d unsupported", a->act_dtype);
    return B2L_E_UNSUPPORTED;
  }
  if (n_chunks > 1) {   // local end states, combine, then the outputs below start from the workspace
    if (cpl == 2) { if (bf) B2L_SCAN_LAUNCH(0, __nv_bfloat16, 1, 2, 4); else B2L_SCAN_LAUNCH(0, float, 1, 2, 5); }
    else { if (bf) B2L_SCAN_LAUNCH(0, __nv_bfloat16, 1, 1, 6); else B2L_SCAN_LAUNCH(0, float, 1, 1, 7); }
    B2L_LAUNCH_CHECK("seq_scan_kernel (local states)");
    const size_t n = (size_t)a->heads * a->V * a->K;
    seq_scan_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(*a);
    B2L_LAUNCH_CHECK("seq_scan_combine_kernel");
  }
  if (a->delta) { if (bf) B2L_SCAN_LAUNCH(1, __nv_bfloat16, 0, 1, 0); else B2L_SCAN_LAUNCH(1, float, 0, 1, 1); }
  else if (cpl == 2) { if (bf) B2L_SCAN_LAUNCH(0, __nv_bfloat16, 0, 2, 2); else B2L_SCAN_LAUNCH(0, float, 0, 2, 3); }
  else { if (bf) B2L_SCAN_LAUNCH(0, __nv_bfloat16, 0, 1, 8); else B2L_SCAN_LAUNCH(0, float, 0, 1, 9); }
#undef B2L_SCAN_LAUNCH
  B2L_LAUNCH_CHECK("seq_scan_kernel");
  return 0;
}
