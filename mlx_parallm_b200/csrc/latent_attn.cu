// Attention over a shared low-rank latent: every position stores ONE vector c (rank R) that serves as key and value of all
// heads; the per-head key and value up-projections are folded into the query (before) and the output (after) by b200p_gemm,
// so the cache is read as it is stored.  A sliding window bounds the visible positions.
//   latent_prep_kernel   rms norms of the two down-projections; the key/value latent goes into the cache
//   latent_attn_kernel   one CTA per token and group of heads; keys staged 32 at a time in shared memory; online fp32 softmax
#include "common.cuh"

namespace b200p {

template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int64_t ldp, int q_rank, int kv_rank,
                                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps, T* __restrict__ cq_out,
                                   T* __restrict__ cache, int64_t Tcap, const int32_t* __restrict__ t_row,
                                   const int32_t* __restrict__ t_pos) {
  __shared__ float red[2];
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;     // warp 0: query part, warp 1: key/value part
  const float* src = proj + t * ldp + (warp == 0 ? 0 : q_rank);
  const int n = warp == 0 ? q_rank : kv_rank;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncwarp();
  if (n == 0) return;
  const float inv = 1.f / sqrtf(red[warp] / (float)n + eps);
  if (warp == 0) {
    for (int i = lane; i < n; i += 32) cq_out[t * q_rank + i] = Tr<T>::from_f(src[i] * inv * wq[i]);
  } else {
    const int64_t pos = t_pos[t];
    if (pos >= Tcap) return;                                       // the host sizes the cache first; never write outside it
    T* dst = cache + ((int64_t)t_row[t] * Tcap + pos) * kv_rank;
    for (int i = lane; i < n; i += 32) dst[i] = Tr<T>::from_f(src[i] * inv * wkv[i]);
  }
}

constexpr int LA_KEYS = 32;       // keys per staged chunk: one per lane in the score phase
constexpr int LA_MAX_HEADS = 8;   // heads (warps) per CTA
constexpr int LA_MAX_RL = 16;     // latent elements per lane in the output phase: R <= 512

template <typename T>
__global__ void __launch_bounds__(LA_MAX_HEADS * 32)
latent_attn_kernel(const float* __restrict__ q, const T* __restrict__ cache, int64_t Tcap, const int32_t* __restrict__ t_row,
                   const int32_t* __restrict__ t_pos, T* __restrict__ out, int H, int R, int64_t window, float scale) {
  extern __shared__ float sm[];
  const int RS = R + 1;                                            // padded row: lane j reads row j without bank conflicts
  float* cs = sm;                                                  // [LA_KEYS][RS]
  float* qs = sm + LA_KEYS * RS;                                   // [warps][R]
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int h = blockIdx.y * nw + warp;
  const bool head_ok = h < H;
  const int64_t pos = t_pos[t];
  const int64_t lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const T* cbase = cache + (int64_t)t_row[t] * Tcap * R;
  if (head_ok)
    for (int r = lane; r < R; r += 32) qs[warp * R + r] = q[(t * H + h) * R + r];
  float acc[LA_MAX_RL];
#pragma unroll
  for (int i = 0; i < LA_MAX_RL; ++i) acc[i] = 0.f;
  float mx = -INFINITY, den = 0.f;
  for (int64_t j0 = lo; j0 <= pos; j0 += LA_KEYS) {
    const int nk = (int)min((int64_t)LA_KEYS, pos + 1 - j0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * R; idx += blockDim.x) {
      const int kk = idx / R, r = idx % R;
      cs[kk * RS + r] = Tr<T>::to_f(cbase[(j0 + kk) * R + r]);
    }
    __syncthreads();
    if (!head_ok) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* cr = cs + lane * RS;
      const float* qr = qs + warp * R;
      float d = 0.f;
      for (int r = 0; r < R; ++r) d = fmaf(qr[r], cr[r], d);
      s = d * scale;
    }
    const float cmx = warp_max(s);
    const float nmx = fmaxf(mx, cmx);
    const float corr = __expf(mx - nmx);                           // 0 on the first chunk (mx = -inf)
    const float p = lane < nk ? __expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int i = 0; i < LA_MAX_RL; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const float* cr = cs + kk * RS;
#pragma unroll
      for (int i = 0; i < LA_MAX_RL; ++i) {
        const int r = i * 32 + lane;
        if (r < R) acc[i] = fmaf(pk, cr[r], acc[i]);
      }
    }
  }
  if (!head_ok) return;
  const float inv = 1.f / den;
#pragma unroll
  for (int i = 0; i < LA_MAX_RL; ++i) {
    const int r = i * 32 + lane;
    if (r < R) out[(t * H + h) * R + r] = Tr<T>::from_f(acc[i] * inv);
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_latent_prep(const float* proj, int64_t ldp, int q_rank, int kv_rank, const float* wq, const float* wkv,
                                 float eps, void* cq_out, void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                                 int64_t M, int dtype, void* stream) {
  B200P_REQUIRE(proj && wq && cq_out && q_rank > 0 && kv_rank >= 0, B200P_ERR_ARG, "null pointer or bad rank");
  B200P_REQUIRE(kv_rank == 0 || (wkv && cache && t_row && t_pos && Tcap > 0), B200P_ERR_ARG, "the key/value latent needs its cache");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (latent_prep_kernel<T><<<(unsigned)M, 64, 0, (cudaStream_t)stream>>>(
      proj, ldp, q_rank, kv_rank, wq, wkv, eps, (T*)cq_out, (T*)cache, Tcap, t_row, t_pos)));
  B200P_LAUNCH_CHECK("latent_prep_kernel");
  return B200P_OK;
}

template <typename T>
static int latent_attn_launch(const float* q, const void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, void* out,
                              int64_t M, int H, int R, int64_t window, float scale, cudaStream_t st) {
  const int nw = H < LA_MAX_HEADS ? H : LA_MAX_HEADS;
  const size_t smem = ((size_t)LA_KEYS * (R + 1) + (size_t)nw * R) * sizeof(float);
  auto kern = latent_attn_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(latent_attn_kernel)");
  }
  dim3 grid((unsigned)M, (unsigned)((H + nw - 1) / nw));
  kern<<<grid, nw * 32, smem, st>>>(q, (const T*)cache, Tcap, t_row, t_pos, (T*)out, H, R, window, scale);
  B200P_LAUNCH_CHECK("latent_attn_kernel");
  return B200P_OK;
}

extern "C" int b200p_latent_attn(const float* q, const void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                                 void* out, int64_t M, int H, int R, int64_t window, float scale, int dtype, void* stream) {
  B200P_REQUIRE(q && cache && t_row && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && R > 0 && R <= 32 * LA_MAX_RL, B200P_ERR_ARG, "latent rank must be in [1, %d]", 32 * LA_MAX_RL);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case B200P_F32: return latent_attn_launch<float>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    case B200P_F16: return latent_attn_launch<__half>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    case B200P_BF16: return latent_attn_launch<__nv_bfloat16>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}
