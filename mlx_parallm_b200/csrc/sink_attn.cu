// Causal attention over a ragged batch for designs without a positional rotation: grouped query heads, separate key and value
// sizes, rms-normed queries and keys, a query temperature that depends on the position, a bias linear in the distance
// (score - slope_h (i - j)) and a learned per-head "sink" that joins the softmax denominator without a key or a value.
//   sink_attn_prep_kernel   norms, temperature and scale on q; normed k and v into the cache at (row, position)     (per token)
//   sink_attn_kernel        one token x the query heads of one key/value head, fp32 throughout, any sizes           (per token)
//   sink_attn_tile_kernel   16 query rows per warp on mma.sync, 64-key chunks staged once for the heads of a group   (16-bit caches)
// The softmax starts from the sink: running maximum = sink, running sum = 1 (the sink's own term), accumulator = 0; every key
// then joins by the usual online update, so a query that sees few keys is damped exactly as the definition says.
// Every option is a parameter: no norm (weights NULL), no temperature (coef 0), no bias (slope_log2 0), no sink (NULL).
#include "common.cuh"
#include "mma_util.cuh"

namespace b200p {

// slope of head h: 2^(slope_log2 * (h + 1) / H); slope_log2 = 0 means no bias
__device__ __forceinline__ float head_slope(float slope_log2, int h, int H) {
  return slope_log2 == 0.f ? 0.f : exp2f(slope_log2 * (float)(h + 1) / (float)H);
}

template <typename T>
__global__ void sink_attn_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v,
                                      const float* __restrict__ wq, const float* __restrict__ wk, float eps, float scale,
                                      float temp_coef, float temp_every, float* __restrict__ q_out, T* __restrict__ kcache,
                                      T* __restrict__ vcache, int64_t Tcap, const int32_t* __restrict__ t_row,
                                      const int32_t* __restrict__ t_pos, int H, int G, int dk, int dv) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float* pt = proj + t * ldp;
  const int64_t pos = t_pos[t], row = t_row[t];
  float qmul = scale;
  if (temp_coef != 0.f) qmul *= 1.f + temp_coef * logf(floorf((float)(pos + 1) / temp_every) + 1.f);
  const bool in_cache = pos < Tcap;                                // the host sizes the cache first; never write outside it
  for (int hd = warp; hd < H + G; hd += nw) {                      // query heads, then key heads
    const bool is_q = hd < H;
    const float* src = is_q ? pt + col_q + (int64_t)hd * dk : pt + col_k + (int64_t)(hd - H) * dk;
    const float* w = is_q ? wq : wk;
    float inv = 1.f;
    if (w) {
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)dk + eps);
    }
    if (is_q) {
      float* dst = q_out + (t * H + hd) * dk;
      for (int i = lane; i < dk; i += 32) dst[i] = src[i] * inv * (w ? w[i] : 1.f) * qmul;
    } else if (in_cache) {
      T* dst = kcache + ((row * G + (hd - H)) * Tcap + pos) * dk;
      for (int i = lane; i < dk; i += 32) dst[i] = Tr<T>::from_f(src[i] * inv * (w ? w[i] : 1.f));
    }
  }
  if (in_cache) {
    for (int c = threadIdx.x; c < G * dv; c += blockDim.x) {
      const int g = c / dv, i = c % dv;
      vcache[((row * G + g) * Tcap + pos) * dv + i] = Tr<T>::from_f(pt[col_v + c]);
    }
  }
}

constexpr int SA_KEYS = 32;        // keys per staged chunk: one per lane in the score phase
constexpr int SA_MAX_HEADS = 8;    // query heads (warps) per CTA
constexpr int SA_MAX_VL = 16;      // value elements per lane: dv <= 512

// CTA = (token t, key/value head g, block of up to 8 of its query heads); warp = query head.
template <typename T>
__global__ void __launch_bounds__(SA_MAX_HEADS * 32)
sink_attn_kernel(const float* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache, int64_t Tcap,
                 const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, const float* __restrict__ sink,
                 float slope_log2, T* __restrict__ out, int64_t ld_out, float out_scale, int H, int G, int dk, int dv) {
  extern __shared__ float sa_sm[];
  const int KS = dk + 1;                                           // padded row: lane j reads row j without bank conflicts
  float* ks = sa_sm;                                               // [SA_KEYS][KS]
  float* vs = ks + SA_KEYS * KS;                                   // [SA_KEYS][dv]
  float* qs = vs + SA_KEYS * dv;                                   // [warps][dk]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y, per = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int hl = blockIdx.z * nw + warp;                           // head inside the group
  const bool head_ok = hl < per;
  const int h = g * per + hl;
  const int64_t pos = t_pos[t];
  const T* kb = kcache + ((int64_t)t_row[t] * G + g) * Tcap * dk;
  const T* vb = vcache + ((int64_t)t_row[t] * G + g) * Tcap * dv;
  if (head_ok)
    for (int i = lane; i < dk; i += 32) qs[warp * dk + i] = q[(t * H + h) * dk + i];
  const float slope = head_ok ? head_slope(slope_log2, h, H) : 0.f;
  float acc[SA_MAX_VL];
#pragma unroll
  for (int i = 0; i < SA_MAX_VL; ++i) acc[i] = 0.f;
  float mx = (head_ok && sink) ? sink[h] : -INFINITY;
  float den = (head_ok && sink) ? 1.f : 0.f;
  for (int64_t j0 = 0; j0 <= pos; j0 += SA_KEYS) {
    const int nk = (int)min((int64_t)SA_KEYS, pos + 1 - j0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * dk; idx += blockDim.x) {
      const int kk = idx / dk, i = idx % dk;
      ks[kk * KS + i] = Tr<T>::to_f(kb[(j0 + kk) * dk + i]);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += blockDim.x) vs[idx] = Tr<T>::to_f(vb[j0 * dv + idx]);
    __syncthreads();
    if (!head_ok) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * KS;
      const float* qr = qs + warp * dk;
      float d = 0.f;
      for (int i = 0; i < dk; ++i) d = fmaf(qr[i], kr[i], d);
      s = d - slope * (float)(pos - (j0 + lane));
    }
    const float nmx = fmaxf(mx, warp_max(s));
    const float corr = __expf(mx - nmx);                           // 0 on the first chunk without a sink (mx = -inf)
    const float p = lane < nk ? __expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int i = 0; i < SA_MAX_VL; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const float* vr = vs + kk * dv;
#pragma unroll
      for (int i = 0; i < SA_MAX_VL; ++i) {
        const int c = i * 32 + lane;
        if (c < dv) acc[i] = fmaf(pk, vr[c], acc[i]);
      }
    }
  }
  if (!head_ok) return;
  const float inv = out_scale / den;
#pragma unroll
  for (int i = 0; i < SA_MAX_VL; ++i) {
    const int c = i * 32 + lane;
    if (c < dv) out[t * ld_out + (int64_t)h * dv + c] = Tr<T>::from_f(acc[i] * inv);
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_sink_attn_prep(const float* proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v, const float* wq,
                                    const float* wk, float eps, float scale, float temp_coef, float temp_every, float* q_out,
                                    void* kcache, void* vcache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, int64_t M,
                                    int H, int G, int dk, int dv, int dtype, void* stream) {
  B200P_REQUIRE(proj && q_out && kcache && vcache && t_row && t_pos, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(temp_coef == 0.f || temp_every > 0.f, B200P_ERR_ARG, "the query temperature needs a positive block length");
  if (M == 0) return B200P_OK;
  const unsigned threads = (H + G) >= 8 ? 256 : 128;
  B200P_DISPATCH_DTYPE(dtype, T, (sink_attn_prep_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      proj, ldp, col_q, col_k, col_v, wq, wk, eps, scale, temp_coef, temp_every, q_out, (T*)kcache, (T*)vcache, Tcap, t_row, t_pos,
      H, G, dk, dv)));
  B200P_LAUNCH_CHECK("sink_attn_prep_kernel");
  return B200P_OK;
}

template <typename T>
static int sink_attn_generic(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                             const int32_t* t_pos, const float* sink, float slope_log2, void* out, int64_t ld_out, float out_scale,
                             int64_t M, int H, int G, int dk, int dv, cudaStream_t st) {
  const int per = H / G, nw = per < SA_MAX_HEADS ? per : SA_MAX_HEADS;
  const size_t smem = ((size_t)SA_KEYS * (dk + 1) + (size_t)SA_KEYS * dv + (size_t)nw * dk) * sizeof(float);
  auto kern = sink_attn_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(sink_attn_kernel)");
  }
  dim3 grid((unsigned)M, (unsigned)G, (unsigned)((per + nw - 1) / nw));
  kern<<<grid, nw * 32, smem, st>>>(q, (const T*)kcache, (const T*)vcache, Tcap, t_row, t_pos, sink, slope_log2, (T*)out, ld_out,
                                    out_scale, H, G, dk, dv);
  B200P_LAUNCH_CHECK("sink_attn_kernel");
  return B200P_OK;
}

extern "C" int b200p_sink_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                               const int32_t* t_pos, const float* sink, float slope_log2, void* out, int64_t ld_out,
                               float out_scale, int64_t M, int H, int G, int dk, int dv, int dtype, void* stream) {
  B200P_REQUIRE(q && kcache && vcache && t_row && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && G < 65536 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(dv <= 32 * SA_MAX_VL && dk <= 1024, B200P_ERR_ARG, "value size above %d or key size above 1024 is not built",
                32 * SA_MAX_VL);
  B200P_REQUIRE(ld_out >= (int64_t)H * dv, B200P_ERR_ARG, "output rows are shorter than the heads");
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case B200P_F32: return sink_attn_generic<float>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st);
    case B200P_F16: return sink_attn_generic<__half>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st);
    case B200P_BF16: return sink_attn_generic<__nv_bfloat16>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}
