// Sliding-window softmax attention over a paged key/value cache, without rotation: positions enter through a bias that depends on
// the distance between query and key only. Per cached token one row [kv_heads * dim keys | kv_heads * vdim values].
//
//   omc_qk_norm_kv_store: the rows of a step -> normed queries, and normed keys + values appended to the pages
//   omc_window_attn:      score = (q . k) * scale -> softcap * tanh(score / softcap) -> + dist_bias[i - j][head] -> softmax over the
//                         keys j with 0 <= i - j < window -> weighted sum of values
// The distance bias arrives as a table [window, heads] that the host builds (here from a bucketed learned table; any function of
// the distance fits). Prompt portions and decoded tokens are one case: row t at position pos[t] of slot[t] reads the cached
// entries max(0, pos - window + 1) .. pos of its slot, which the store kernel of the same step has written.
// The plain kernel: fp32 arithmetic, one CTA per (row, head), a warp per key, lanes across the head dimension.
#include <math.h>

#include "seq_common.cuh"

namespace omc {

constexpr int kWinWarps = 4;
constexpr int kWinMaxPerLane = 8;  // value width up to 256

// One CTA per row. q: RMS norm over all H * d query columns with a plain weight -> q_out. k likewise -> page; v copied -> page.
template <typename TW, typename TC>
__global__ void __launch_bounds__(256) qk_norm_kv_store_kernel(const float* __restrict__ q, long long ldq, int nq,
                                                               const TW* __restrict__ wq, const float* __restrict__ k, long long ldk,
                                                               int nk, const TW* __restrict__ wk, const float* __restrict__ v,
                                                               long long ldv, int nv, float eps, const int32_t* __restrict__ pos,
                                                               const int32_t* __restrict__ slot, const int32_t* __restrict__ block_table,
                                                               int max_pages, int page_size, TC* __restrict__ pool,
                                                               TC* __restrict__ q_out, long long ldqo) {
  __shared__ float red[33];
  const long long t = blockIdx.x;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  TC* dst = pool + ((long long)page * page_size + p % page_size) * (nk + nv);
  float ss = 0.f;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) {
    const float x = q[t * ldq + c];
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, red);
  float rstd = 1.f / sqrtf(ss / (float)nq + eps);
  for (int c = threadIdx.x; c < nq; c += blockDim.x) stf(q_out + t * ldqo + c, q[t * ldq + c] * rstd * ldf(wq + c));
  ss = 0.f;
  for (int c = threadIdx.x; c < nk; c += blockDim.x) {
    const float x = k[t * ldk + c];
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, red);
  rstd = 1.f / sqrtf(ss / (float)nk + eps);
  for (int c = threadIdx.x; c < nk; c += blockDim.x) stf(dst + c, k[t * ldk + c] * rstd * ldf(wk + c));
  for (int c = threadIdx.x; c < nv; c += blockDim.x) stf(dst + nk + c, v[t * ldv + c]);
}

template <typename TQ, typename TC, typename TY>
__global__ void __launch_bounds__(kWinWarps * 32) window_attn_kernel(const TQ* __restrict__ q, long long ldq, int H, int G, int d,
                                                                     int dv, const TC* __restrict__ pool,
                                                                     const int32_t* __restrict__ block_table, int max_pages,
                                                                     int page_size, const int32_t* __restrict__ pos,
                                                                     const int32_t* __restrict__ slot, int window, float scale,
                                                                     float softcap, const float* __restrict__ dist_bias,
                                                                     TY* __restrict__ out, long long ldo) {
  extern __shared__ float sm[];  // q [d] | acc [warps][dv] | m [warps] | l [warps]
  const int t = blockIdx.x, h = blockIdx.y, kvh = h / (H / G);
  float* sq = sm;
  float* sacc = sm + d;
  float* s_m = sacc + kWinWarps * dv;
  float* s_l = s_m + kWinWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < d; c += blockDim.x) sq[c] = ldf(q + (long long)t * ldq + h * d + c);
  __syncthreads();
  const int p = pos[t];
  const int first = max(0, p - window + 1);
  const int32_t* bt = block_table + (long long)slot[t] * max_pages;
  const int W = G * (d + dv);
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  float m = -INFINITY, l = 0.f;
  float acc[kWinMaxPerLane];
#pragma unroll
  for (int i = 0; i < kWinMaxPerLane; ++i) acc[i] = 0.f;
  for (int j = first + warp; j <= p; j += kWinWarps) {
    const TC* row = pool + ((long long)bt[j / page_size] * page_size + j % page_size) * W;
    const TC* kr = row + kvh * d;
    const TC* vr = row + G * d + kvh * dv;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s = fmaf(sq[c], ldf(kr + c), s);
    s = seq_warp_sum(s) * scale;
    if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
    if (dist_bias != nullptr) s += dist_bias[(long long)(p - j) * H + h];
    const float mn = fmaxf(m, s);
    const float corr = expf(m - mn), pj = expf(s - mn);  // m = -inf on the first key: corr = 0
    l = l * corr + pj;
#pragma unroll
    for (int i = 0; i < kWinMaxPerLane; ++i) {
      const int c = lane + 32 * i;
      if (c < dv) acc[i] = acc[i] * corr + pj * ldf(vr + c);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kWinMaxPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) sacc[warp * dv + c] = acc[i];
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  float mt = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWinWarps; ++w) mt = fmaxf(mt, s_m[w]);
  float lt = 0.f;
  float f[kWinWarps];
#pragma unroll
  for (int w = 0; w < kWinWarps; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - mt);
    lt += s_l[w] * f[w];
  }
  const float inv = 1.f / lt;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kWinWarps; ++w) o += sacc[w * dv + c] * f[w];
    stf(out + (long long)t * ldo + h * dv + c, o * inv);
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_qk_norm_kv_store(const float* q, long long ldq, int nq, const void* wq, const float* k, long long ldk, int nk,
                                    const void* wk, int w_dt, const float* v, long long ldv, int nv, float eps, int T,
                                    const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size,
                                    void* pool, void* q_out, long long ldqo, int dt, void* stream) {
  if (q == nullptr || wq == nullptr || k == nullptr || wk == nullptr || v == nullptr || pos == nullptr || slot == nullptr ||
      block_table == nullptr || pool == nullptr || q_out == nullptr || T < 0 || nq <= 0 || nk <= 0 || nv <= 0 || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_qk_norm_kv_store: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(dt, TC, {
    qk_norm_kv_store_kernel<TW, TC><<<T, 256, 0, st>>>(q, ldq, nq, static_cast<const TW*>(wq), k, ldk, nk, static_cast<const TW*>(wk), v,
                                                       ldv, nv, eps, pos, slot, block_table, max_pages, page_size,
                                                       static_cast<TC*>(pool), static_cast<TC*>(q_out), ldqo);
  }))
  return check_launch("omc_qk_norm_kv_store");
}

extern "C" int omc_window_attn(const void* q, long long ldq, int T, int H, int G, int d, int dv, const void* pool, int dt,
                               const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot,
                               int window, float scale, float softcap, const float* dist_bias, void* out, int out_dt, long long ldo,
                               void* stream) {
  if (q == nullptr || pool == nullptr || block_table == nullptr || pos == nullptr || slot == nullptr || out == nullptr || T < 0 ||
      H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || window < 1 || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_window_attn: bad argument");
  if (T == 0) return OMC_OK;
  if (dv > 32 * kWinMaxPerLane) return set_error(OMC_ERR_SHAPE, "omc_window_attn: value width above 256");
  if (H > 65535) return set_error(OMC_ERR_SHAPE, "omc_window_attn: more than 65535 heads");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(float) * ((size_t)d + (size_t)kWinWarps * dv + 2 * kWinWarps);
  if (smem > 48 * 1024) return set_error(OMC_ERR_SHAPE, "omc_window_attn: head width too large");
  OMC_DT_SWITCH(dt, TC, OMC_DT_SWITCH(out_dt, TY, {
    window_attn_kernel<TC, TC, TY><<<dim3(T, H), kWinWarps * 32, smem, st>>>(static_cast<const TC*>(q), ldq, H, G, d, dv,
                                                                            static_cast<const TC*>(pool), block_table, max_pages,
                                                                            page_size, pos, slot, window, scale, softcap, dist_bias,
                                                                            static_cast<TY*>(out), ldo);
  }))
  return check_launch("omc_window_attn");
}
