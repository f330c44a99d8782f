// Gated delta rule (a linear-attention layer with a per-head matrix state S [dk, dv] that is decayed, corrected towards the
// current value along the current key and read with the current query), as four kernels over a ragged batch:
//   delta_prep_kernel         short causal convolution + silu of q, k, v; unit q / k per head; beta and decay   (per token)
//   delta_conv_commit_kernel  the convolution's carried inputs                                                   (per entry)
//   delta_scan_kernel         the recurrence, fp32, token by token; four lanes per pair of state columns           (per entry, head)
//   delta_out_kernel          per-head rms norm * weight * silu(gate)                                            (per token)
// The same kernels carry the variants other designs use: a decay per head AND key channel (a row of S each), a gate that is a
// sigmoid of a separate tensor, and the plain decayed accumulation S <- g S + k v^T (linear attention with a constant decay,
// fed by linear_attn_prep_kernel).
// Prompts and single decoded tokens run the SAME scan kernel in the same summation order, so a prompt cut into portions gives
// the same numbers as one pass.
#include "common.cuh"

namespace b200p {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int DELTA_MAX_TAPS = 16;

template <int NT>
__global__ void __launch_bounds__(NT)
delta_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_b, const float* __restrict__ a, int64_t lda, int dper,
                  const float* __restrict__ conv_w,
                  const float* __restrict__ conv_state, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                  const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, const int32_t* __restrict__ t_off,
                  float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vout, float* __restrict__ beta,
                  float* __restrict__ decay, int H, int KH, int dk, int dv, int taps) {
  extern __shared__ float qk[];                      // conv + silu of the q and k channels of this token
  const int64_t t = blockIdx.x;
  const int Cqk = 2 * KH * dk, C = Cqk + H * dv;
  const int row = t_row[t], pos = t_pos[t], off = t_off[t];
  const float* pt = proj + t * ldp;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {                 // tap j multiplies the input d = taps-1-j tokens back
      const int d = taps - 1 - j;
      float in;
      if (d > pos) in = 0.f;                         // before the sequence
      else if (d <= off) in = pt[c - (int64_t)d * ldp];
      else in = conv_state[((int64_t)row * (taps - 1) + (taps - 1 + off - d)) * C + c];
      acc = fmaf(conv_w[(int64_t)c * taps + j], in, acc);
    }
    const float a = silu_f(acc);
    if (c < Cqk) qk[c] = a;
    else vout[t * (int64_t)(H * dv) + (c - Cqk)] = a;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int hd = warp; hd < 2 * KH; hd += nw) {       // heads 0..KH-1 of q, then of k
    const float* src = qk + hd * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    float inv = 1.f / sqrtf(ss + 1e-6f);
    float* dst;
    if (hd < KH) { inv *= 1.f / sqrtf((float)dk); dst = qn + t * (int64_t)(KH * dk) + hd * dk; }
    else dst = kn + t * (int64_t)(KH * dk) + (hd - KH) * dk;
    for (int i = lane; i < dk; i += 32) dst[i] = src[i] * inv;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) beta[t * H + h] = 1.f / (1.f + expf(-pt[col_b + h]));
  // dper decays per head (1: the whole state of a head; dk: one per key channel), each with its own step input and bias
  const int nd = H * dper;
  const float* at = a + t * lda;
  for (int i = threadIdx.x; i < nd; i += blockDim.x)
    decay[t * (int64_t)nd + i] = expf(-expf(A_log[i / dper]) * softplus_f(at[i] + dt_bias[i]));
}

// Inputs of the plain decayed accumulation: q, k, v = silu of their projections (columns [0, Cqk), [Cqk, 2 Cqk), [2 Cqk, ..) of
// proj), and the constant per-head decay repeated for every token so that the scan reads it like a computed one.
__global__ void linear_attn_prep_kernel(const float* __restrict__ proj, int64_t ldp, const float* __restrict__ head_decay,
                                        float* __restrict__ q, float* __restrict__ k, float* __restrict__ v,
                                        float* __restrict__ decay, int H, int Cqk, int Cv) {
  const int64_t t = blockIdx.x;
  const float* pt = proj + t * ldp;
  for (int c = threadIdx.x; c < 2 * Cqk + Cv; c += blockDim.x) {
    const float a = silu_f(pt[c]);
    if (c < Cqk) q[t * Cqk + c] = a;
    else if (c < 2 * Cqk) k[t * Cqk + (c - Cqk)] = a;
    else v[t * (int64_t)Cv + (c - 2 * Cqk)] = a;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) decay[t * H + h] = head_decay[h];
}

__global__ void delta_conv_commit_kernel(const float* __restrict__ proj, int64_t ldp, float* __restrict__ conv_state,
                                         const int32_t* __restrict__ cu, const int32_t* __restrict__ rows, int64_t C, int taps) {
  const int e = blockIdx.y;
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int n = cu[e + 1] - cu[e];
  if (c >= C || n <= 0) return;
  float* st = conv_state + (int64_t)rows[e] * (taps - 1) * C + c;
  float keep[DELTA_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < DELTA_MAX_TAPS; ++i) {
    if (i < taps - 1) {
      const int rel = n - (taps - 1) + i;            // input i of the new state, counted from the portion's first token
      keep[i] = rel >= 0 ? proj[((int64_t)cu[e] + rel) * ldp + c] : st[(int64_t)(i + n) * C];
    }
  }
#pragma unroll
  for (int i = 0; i < DELTA_MAX_TAPS; ++i)
    if (i < taps - 1) st[(int64_t)i * C] = keep[i];
}

constexpr int DS_THREADS = 128;
// lanes that share a state column (lane l keeps rows [l * dkp / lanes, (l + 1) * dkp / lanes) in registers): at most 32 rows each
constexpr int ds_lanes(int dkp) { return dkp <= 128 ? 4 : dkp / 32; }
constexpr int ds_cols(int dkp) { return 2 * DS_THREADS / ds_lanes(dkp); }      // state columns per CTA: two per column slot

// dk padded to DKP = 32 ... 512.  A thread owns a part (a quarter up to 128 rows, 32 rows beyond) of the rows of TWO state
// columns, kept as float2 pairs: a head's value size of 128 is spread over 256 threads instead of 128, every q / k element read
// from shared memory serves two columns (shared-memory wavefronts, not arithmetic, bound the one-column variants), and the
// packed fp32 instructions of sm_100 (FMUL2 / FFMA2: both halves rounded like the scalar operation) update both columns at
// once.  Each reduction over dk is as much shorter plus log2(lanes) exchanges between the lanes.  q and k of CHUNK tokens are
// staged in shared memory with every lane's part padded by 16 bytes, so the lanes' 128-bit reads fall into different banks.
// MODE 0: delta rule, one decay per head and token; 1: delta rule, one decay per head, key channel and token (decay
// [M, H, dk]); 2: no correction, S <- g S + k v^T (one decay per head and token; beta unused).
template <int DKP, int MODE>
__global__ void __launch_bounds__(DS_THREADS)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                  const int32_t* __restrict__ cu, const int32_t* __restrict__ rows, const int32_t* __restrict__ lengths,
                  float* __restrict__ o, int H, int KH, int dk, int dv) {
  constexpr int DS_LANES = ds_lanes(DKP), DS_SLOTS = DS_THREADS / DS_LANES, DS_COLS = 2 * DS_SLOTS;
  constexpr int SEG = DKP / DS_LANES;                            // state rows per lane
  constexpr int CHUNK = DKP <= 128 ? 8 : 1024 / DKP;             // tokens staged at a time
  constexpr int LDK = DKP + 4 * DS_LANES;                        // padded row of the staging buffers
  constexpr int PF = CHUNK * DKP / DS_THREADS;                   // q / k elements each thread stages per chunk
  constexpr int PV = (CHUNK * DS_COLS + DS_THREADS - 1) / DS_THREADS;
  __shared__ __align__(16) float ks[2][CHUNK][LDK], qs[2][CHUNK][LDK];
  __shared__ __align__(16) float gc[MODE == 1 ? 2 : 1][MODE == 1 ? CHUNK : 1][MODE == 1 ? LDK : 4];     // per-channel decays
  __shared__ float vs[2][CHUNK][DS_COLS], gs[2][CHUNK], bs[2][CHUNK];
  const int e = blockIdx.x, h = blockIdx.y;
  const int l = threadIdx.x & (DS_LANES - 1), slot = threadIdx.x / DS_LANES;
  const int j0 = blockIdx.z * DS_COLS + slot, j1 = j0 + DS_SLOTS;                // this thread's two state columns
  const bool live0 = j0 < dv, live1 = j1 < dv;
  const int t0 = cu[e], t1 = cu[e + 1];
  if (t1 <= t0) return;
  const int row = rows[e];
  const int kh = h / (H / KH);
  float2 S2[SEG];                                                // .x: column j0, .y: column j1
  float* sp = state + (((int64_t)row * H + h) * dk + l * SEG) * dv;
  const bool fresh = lengths[row] == 0;                          // first token of a sequence: the state starts at zero
#pragma unroll
  for (int i = 0; i < SEG; ++i) {
    const bool in = !fresh && l * SEG + i < dk;
    S2[i].x = (in && live0) ? sp[(int64_t)i * dv + j0] : 0.f;
    S2[i].y = (in && live1) ? sp[(int64_t)i * dv + j1] : 0.f;
  }
  // The next chunk's inputs are fetched into registers while the current chunk runs out of shared memory, then parked in the
  // other buffer: the recurrence never waits for global memory.
  float pk[PF], pq[PF], pv[PV], pg = 0.f, pb = 0.f;
  float pgc[MODE == 1 ? PF : 1];
  auto fetch = [&](int tc) {
    const int nt = min(CHUNK, t1 - tc);
#pragma unroll
    for (int r = 0; r < PF; ++r) {
      const int idx = threadIdx.x + r * DS_THREADS, tt = idx / DKP, i = idx % DKP;
      const bool ok = tt < nt && i < dk;
      const int64_t src = ((int64_t)(tc + tt) * KH + kh) * dk + i;
      pk[r] = ok ? kn[src] : 0.f;
      pq[r] = ok ? qn[src] : 0.f;
      if constexpr (MODE == 1) pgc[r] = ok ? decay[((int64_t)(tc + tt) * H + h) * dk + i] : 1.f;
    }
#pragma unroll
    for (int r = 0; r < PV; ++r) {
      const int idx = threadIdx.x + r * DS_THREADS, tt = idx / DS_COLS, c = blockIdx.z * DS_COLS + idx % DS_COLS;
      pv[r] = (tt < nt && c < dv) ? v[((int64_t)(tc + tt) * H + h) * dv + c] : 0.f;
    }
    if (threadIdx.x < nt) {
      if constexpr (MODE != 1) pg = decay[(int64_t)(tc + threadIdx.x) * H + h];
      if constexpr (MODE != 2) pb = beta[(int64_t)(tc + threadIdx.x) * H + h];
    }
  };
  auto park = [&](int buf) {
#pragma unroll
    for (int r = 0; r < PF; ++r) {
      const int idx = threadIdx.x + r * DS_THREADS, tt = idx / DKP, i = idx % DKP;
      ks[buf][tt][i + (i / SEG) * 4] = pk[r];
      qs[buf][tt][i + (i / SEG) * 4] = pq[r];
      if constexpr (MODE == 1) gc[buf][tt][i + (i / SEG) * 4] = pgc[r];
    }
#pragma unroll
    for (int r = 0; r < PV; ++r) {
      const int idx = threadIdx.x + r * DS_THREADS;
      if (idx < CHUNK * DS_COLS) vs[buf][idx / DS_COLS][idx % DS_COLS] = pv[r];
    }
    if (threadIdx.x < CHUNK) { gs[buf][threadIdx.x] = pg; bs[buf][threadIdx.x] = pb; }
  };
  fetch(t0);
  park(0);
  __syncthreads();
  int buf = 0;
  for (int tc = t0; tc < t1; tc += CHUNK, buf ^= 1) {
    const int nt = min(CHUNK, t1 - tc);
    const bool more = tc + CHUNK < t1;
    if (more) fetch(tc + CHUNK);
    for (int tt = 0; tt < nt; ++tt) {
      const float2 v2 = make_float2(vs[buf][tt][slot], vs[buf][tt][slot + DS_SLOTS]);
      const float g = gs[buf][tt], b = bs[buf][tt];
      const float2 g2 = make_float2(g, g);
      const float* kp = &ks[buf][tt][l * (SEG + 4)];
      const float* qp = &qs[buf][tt][l * (SEG + 4)];
      // both reductions run as four interleaved partial sums per lane (rows i mod 4), combined in a fixed order and then across
      // the lanes by exchanges: short dependency chains, and the same numbers whether a token arrives in a prompt or
      // alone
      float2 d[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) d[a] = make_float2(0.f, 0.f);
      float4 kr[SEG / 4];                                        // the keys stay in registers for the update below
#pragma unroll
      for (int i = 0; i < SEG; i += 4) {
        const float4 k4 = kr[i / 4] = *reinterpret_cast<const float4*>(kp + i);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
        float gg[4] = {g, g, g, g};
        if constexpr (MODE == 1) {
          const float4 g4 = *reinterpret_cast<const float4*>(&gc[buf][tt][l * (SEG + 4) + i]);
          gg[0] = g4.x, gg[1] = g4.y, gg[2] = g4.z, gg[3] = g4.w;
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          S2[i + a] = __fmul2_rn(S2[i + a], MODE == 1 ? make_float2(gg[a], gg[a]) : g2);
          if constexpr (MODE != 2) d[a] = __ffma2_rn(S2[i + a], make_float2(kk[a], kk[a]), d[a]);
        }
      }
      float2 u2 = v2;
      if constexpr (MODE != 2) {
        float dx = (d[0].x + d[1].x) + (d[2].x + d[3].x), dy = (d[0].y + d[1].y) + (d[2].y + d[3].y);
#pragma unroll
        for (int m = 1; m < DS_LANES; m <<= 1) {
          dx += __shfl_xor_sync(0xffffffffu, dx, m);
          dy += __shfl_xor_sync(0xffffffffu, dy, m);
        }
        u2 = make_float2(b * (v2.x - dx), b * (v2.y - dy));
      }
      float2 oa[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) oa[a] = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < SEG; i += 4) {
        const float4 k4 = kr[i / 4];
        const float4 q4 = *reinterpret_cast<const float4*>(qp + i);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          S2[i + a] = __ffma2_rn(make_float2(kk[a], kk[a]), u2, S2[i + a]);
          oa[a] = __ffma2_rn(S2[i + a], make_float2(qq[a], qq[a]), oa[a]);
        }
      }
      float ox = (oa[0].x + oa[1].x) + (oa[2].x + oa[3].x), oy = (oa[0].y + oa[1].y) + (oa[2].y + oa[3].y);
#pragma unroll
      for (int m = 1; m < DS_LANES; m <<= 1) {
        ox += __shfl_xor_sync(0xffffffffu, ox, m);
        oy += __shfl_xor_sync(0xffffffffu, oy, m);
      }
      if (l == 0) {
        float* op = o + ((int64_t)(tc + tt) * H + h) * dv;
        if (live0) op[j0] = ox;
        if (live1) op[j1] = oy;
      }
    }
    if (more) park(buf ^ 1);          // the other buffer was last read in the previous iteration, before its closing barrier
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < SEG; ++i) {
    if (l * SEG + i < dk) {
      if (live0) sp[(int64_t)i * dv + j0] = S2[i].x;
      if (live1) sp[(int64_t)i * dv + j1] = S2[i].y;
    }
  }
}

__device__ __forceinline__ float gate_act_f(float z, int act) { return act == 0 ? silu_f(z) : 1.f / (1.f + expf(-z)); }

// groups of dv values (a head each, or all heads as one group when H == 1) are rms-normed, weighted by norm_w [dv], gated by
// act(gate) (0 silu, 1 sigmoid) and scaled; out rows have stride ld_out
template <typename T>
__global__ void delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t ldg,
                                 const float* __restrict__ norm_w, T* __restrict__ out, int64_t ld_out, int H, int dv, float eps,
                                 int act, float out_scale) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (H == 1) {                                   // one wide group: the whole block sums it, in an order fixed by the block size
    __shared__ float red[32];
    const float* src = o + t * dv;
    const float* g = gate + t * ldg;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += red[i];
    const float inv = out_scale / sqrtf(tot / (float)dv + eps);
    for (int i = threadIdx.x; i < dv; i += blockDim.x)
      out[t * ld_out + i] = Tr<T>::from_f(src[i] * inv * norm_w[i] * gate_act_f(g[i], act));
    return;
  }
  for (int h = warp; h < H; h += nw) {
    const float* src = o + (t * H + h) * dv;
    const float* g = gate + t * ldg + (int64_t)h * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32)
      out[t * ld_out + (int64_t)h * dv + i] = Tr<T>::from_f(src[i] * inv * norm_w[i] * gate_act_f(g[i], act));
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_delta_prep(const float* proj, int64_t ldp, int64_t col_b, const float* a, int64_t lda, int decay_per_head,
                                const float* conv_w, const float* conv_state, const float* A_log, const float* dt_bias, const int32_t* t_row,
                                const int32_t* t_pos, const int32_t* t_off, float* qn, float* kn, float* v, float* beta,
                                float* decay, int64_t M, int H, int KH, int dk, int dv, int taps, void* stream) {
  B200P_REQUIRE(a && (decay_per_head == 1 || decay_per_head == dk), B200P_ERR_ARG, "one decay per head, or one per key channel");
  B200P_REQUIRE(proj && conv_w && conv_state && A_log && dt_bias && t_row && t_pos && t_off && qn && kn && v && beta && decay,
                B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && KH > 0 && H % KH == 0 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(taps >= 1 && taps <= DELTA_MAX_TAPS, B200P_ERR_ARG, "convolution taps must be in [1, %d]", DELTA_MAX_TAPS);
  if (M == 0) return B200P_OK;
  const size_t smem = (size_t)2 * KH * dk * sizeof(float);
  B200P_REQUIRE(smem <= 48 * 1024, B200P_ERR_ARG, "q and k of one token must fit 48 KB of shared memory");
  // a decode batch has few tokens and thousands of channels each: wider blocks shorten the per-thread channel loop
  if (M <= 256)
    delta_prep_kernel<1024><<<(unsigned)M, 1024, smem, (cudaStream_t)stream>>>(proj, ldp, col_b, a, lda, decay_per_head, conv_w, conv_state, A_log, dt_bias, t_row,
                                                                               t_pos, t_off, qn, kn, v, beta, decay, H, KH, dk, dv, taps);
  else
    delta_prep_kernel<256><<<(unsigned)M, 256, smem, (cudaStream_t)stream>>>(proj, ldp, col_b, a, lda, decay_per_head, conv_w, conv_state, A_log, dt_bias, t_row,
                                                                             t_pos, t_off, qn, kn, v, beta, decay, H, KH, dk, dv, taps);
  B200P_LAUNCH_CHECK("delta_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_delta_conv_commit(const float* proj, int64_t ldp, float* conv_state, const int32_t* cu, const int32_t* rows,
                                       int nb, int64_t C, int taps, void* stream) {
  B200P_REQUIRE(proj && conv_state && cu && rows && nb > 0 && nb < 65536, B200P_ERR_ARG, "null pointer or bad batch");
  B200P_REQUIRE(taps >= 1 && taps <= DELTA_MAX_TAPS, B200P_ERR_ARG, "convolution taps must be in [1, %d]", DELTA_MAX_TAPS);
  if (taps == 1) return B200P_OK;
  dim3 grid((unsigned)((C + 127) / 128), (unsigned)nb);
  delta_conv_commit_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(proj, ldp, conv_state, cu, rows, C, taps);
  B200P_LAUNCH_CHECK("delta_conv_commit_kernel");
  return B200P_OK;
}

template <int MODE>
static void delta_scan_launch(dim3 grid, cudaStream_t st, const float* qn, const float* kn, const float* v, const float* beta,
                              const float* decay, float* state, const int32_t* cu, const int32_t* rows, const int32_t* lengths,
                              float* o, int H, int KH, int dk, int dv) {
  const int threads = DS_THREADS;
  if (dk <= 32) delta_scan_kernel<32, MODE><<<grid, threads, 0, st>>>(qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else if (dk <= 64) delta_scan_kernel<64, MODE><<<grid, threads, 0, st>>>(qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else if (dk <= 128) delta_scan_kernel<128, MODE><<<grid, threads, 0, st>>>(qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else if (dk <= 256) delta_scan_kernel<256, MODE><<<grid, threads, 0, st>>>(qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else delta_scan_kernel<512, MODE><<<grid, threads, 0, st>>>(qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
}

extern "C" int b200p_delta_scan(const float* qn, const float* kn, const float* v, const float* beta, const float* decay,
                                float* state, const int32_t* cu, const int32_t* rows, const int32_t* lengths, float* o, int nb,
                                int H, int KH, int dk, int dv, int mode, void* stream) {
  B200P_REQUIRE(qn && kn && v && decay && state && cu && rows && lengths && o, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(mode >= B200P_SCAN_DELTA && mode <= B200P_SCAN_ACCUMULATE, B200P_ERR_ARG, "unknown scan mode %d", mode);
  B200P_REQUIRE(beta || mode == B200P_SCAN_ACCUMULATE, B200P_ERR_ARG, "the delta rule needs beta");
  B200P_REQUIRE(nb > 0 && H > 0 && KH > 0 && H % KH == 0 && H < 65536 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(dk <= 512, B200P_ERR_ARG, "key size %d > 512 is not built", dk);
  const int dkp = dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : dk <= 256 ? 256 : 512, cols = ds_cols(dkp);
  dim3 grid((unsigned)nb, (unsigned)H, (unsigned)((dv + cols - 1) / cols));
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == B200P_SCAN_DELTA) delta_scan_launch<0>(grid, st, qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else if (mode == B200P_SCAN_DELTA_CHANNEL) delta_scan_launch<1>(grid, st, qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  else delta_scan_launch<2>(grid, st, qn, kn, v, beta, decay, state, cu, rows, lengths, o, H, KH, dk, dv);
  B200P_LAUNCH_CHECK("delta_scan_kernel");
  return B200P_OK;
}

extern "C" int b200p_linear_attn_prep(const float* proj, int64_t ldp, const float* head_decay, float* q, float* k, float* v,
                                      float* decay, int64_t M, int H, int dk, int dv, void* stream) {
  B200P_REQUIRE(proj && head_decay && q && k && v && decay && H > 0 && dk > 0 && dv > 0, B200P_ERR_ARG, "null pointer");
  if (M == 0) return B200P_OK;
  linear_attn_prep_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(proj, ldp, head_decay, q, k, v, decay, H, H * dk, H * dv);
  B200P_LAUNCH_CHECK("linear_attn_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_delta_out(const float* o, const float* gate, int64_t ldg, const float* norm_w, void* out, int64_t ld_out,
                               int64_t M, int H, int dv, float eps, int gate_act, float out_scale, int dtype, void* stream) {
  B200P_REQUIRE(o && gate && norm_w && out && H > 0 && dv > 0, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(gate_act == 0 || gate_act == 1, B200P_ERR_ARG, "gate activation: 0 silu, 1 sigmoid");
  B200P_REQUIRE(ld_out >= (int64_t)H * dv, B200P_ERR_ARG, "output rows are shorter than the heads");
  if (M == 0) return B200P_OK;
  const unsigned threads = H == 1 ? (dv >= 1024 ? 256 : 128) : H >= 8 ? 256 : 32 * (unsigned)H;
  B200P_DISPATCH_DTYPE(dtype, T, (delta_out_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      o, gate, ldg, norm_w, (T*)out, ld_out, H, dv, eps, gate_act, out_scale)));
  B200P_LAUNCH_CHECK("delta_out_kernel");
  return B200P_OK;
}
