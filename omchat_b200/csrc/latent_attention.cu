// Latent (compressed key/value) attention over a paged cache.
//
// What is cached per token and layer is ONE row shared by all heads: the normed latent c [r] followed by the rotated key part
// k_rot [dr]. The per-head key / value up-projections are absorbed into the query and the output:
//     score_h(i, j) = (q_h^nope W_uk,h) . c_j + q_h^rot . k_rot_j          o_h(i) = W_uv,h (sum_j p_h(i, j) c_j)
// so the attention kernel is multi-query attention with key width r + dr and value = the first r columns of the same row, and a
// key tile staged once serves as keys and as values. Kernels here:
//   omc_latent_kv_store  one CTA per new row: RMS norm of the latent, pairwise-interleaved rotation of the key part, append to the
//                        row's page (fused norm + rotation + cache write)
//   omc_rotary_q         the rotated query parts, written behind the absorbed part of each head
//   omc_latent_attn      plain kernel, any sizes, fp32 arithmetic: one CTA per (row, head), one warp per key, online softmax with
//                        an optional sink term exp(sink_h) that only enlarges the denominator
// Rows of a step are addressed by (slot, position): a row sees cache entries 0..position of its slot, whether they were written
// by this step or by earlier ones, so portions of prompts and single decoded tokens are the same case.
#include "seq_common.cuh"

namespace omc {

template <typename TW, typename TC>
__global__ void __launch_bounds__(128) latent_kv_store_kernel(const float* __restrict__ dkv, long long ld, int r, int dr,
                                                              const TW* __restrict__ w, float eps, const float* __restrict__ cs,
                                                              int rot_dims, const int32_t* __restrict__ pos,
                                                              const int32_t* __restrict__ slot,
                                                              const int32_t* __restrict__ block_table, int max_pages,
                                                              int page_size, TC* __restrict__ pool) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* row = dkv + (long long)t * ld;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  TC* dst = pool + ((long long)page * page_size + p % page_size) * (r + dr);
  float ss = 0.f;
  for (int c = threadIdx.x; c < r; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)r + eps);
  for (int c = threadIdx.x; c < r; c += blockDim.x) stf(dst + c, row[c] * rstd * ldf(w + c));
  const int half = rot_dims >> 1;
  const float* csr = cs + (long long)p * rot_dims;  // [half][2]
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = row[r + 2 * i], v = row[r + 2 * i + 1], co = csr[2 * i], si = csr[2 * i + 1];
    stf(dst + r + 2 * i, u * co - v * si);
    stf(dst + r + 2 * i + 1, v * co + u * si);
  }
  for (int c = rot_dims + threadIdx.x; c < dr; c += blockDim.x) stf(dst + r + c, row[r + c]);
}

template <typename TQ>
__global__ void __launch_bounds__(128) rotary_q_kernel(const float* __restrict__ q32, long long ldq, int H, int dn, int dr,
                                                       const float* __restrict__ cs, int rot_dims,
                                                       const int32_t* __restrict__ pos, TQ* __restrict__ qcat, int r) {
  const int t = blockIdx.x;
  const float* csr = cs + (long long)pos[t] * rot_dims;
  const int half = rot_dims >> 1;
  for (int h = 0; h < H; ++h) {
    const float* src = q32 + (long long)t * ldq + (long long)h * (dn + dr) + dn;
    TQ* dst = qcat + ((long long)t * H + h) * (r + dr) + r;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float u = src[2 * i], v = src[2 * i + 1], co = csr[2 * i], si = csr[2 * i + 1];
      stf(dst + 2 * i, u * co - v * si);
      stf(dst + 2 * i + 1, v * co + u * si);
    }
    for (int c = rot_dims + threadIdx.x; c < dr; c += blockDim.x) stf(dst + c, src[c]);
  }
}

constexpr int kLatWarps = 4;
constexpr int kLatMaxPerLane = 32;  // r <= 1024

// One CTA per (row, head). Warp w takes keys w, w + 4, ...: lanes split the r + dr columns of the key row for the dot product,
// every lane keeps its share (columns lane, lane + 32, ...) of the running weighted sum of latents. The warps' partial
// (max, sum, accumulator) triples are merged through shared memory at the end.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(kLatWarps * 32) latent_attn_kernel(const TQ* __restrict__ qcat, int H, int r, int dr,
                                                                     const TC* __restrict__ pool,
                                                                     const int32_t* __restrict__ block_table, int max_pages,
                                                                     int page_size, const int32_t* __restrict__ pos,
                                                                     const int32_t* __restrict__ slot,
                                                                     const float* __restrict__ sink, float scale,
                                                                     float* __restrict__ out) {
  extern __shared__ float sm[];  // q [r + dr] | acc [kLatWarps][r] | m [kLatWarps] | l [kLatWarps]
  const int t = blockIdx.x, h = blockIdx.y;
  const int D = r + dr;
  float* sq = sm;
  float* sacc = sm + D;
  float* s_m = sacc + kLatWarps * r;
  float* s_l = s_m + kLatWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TQ* q = qcat + ((long long)t * H + h) * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) sq[c] = ldf(q + c);
  __syncthreads();
  const int n_keys = pos[t] + 1;
  const int32_t* bt = block_table + (long long)slot[t] * max_pages;
  float m = -INFINITY, l = 0.f;
  float acc[kLatMaxPerLane];
#pragma unroll
  for (int i = 0; i < kLatMaxPerLane; ++i) acc[i] = 0.f;
  for (int j = warp; j < n_keys; j += kLatWarps) {
    const TC* kr = pool + ((long long)bt[j / page_size] * page_size + j % page_size) * D;
    float d = 0.f;
    for (int c = lane; c < D; c += 32) d = fmaf(sq[c], ldf(kr + c), d);
    d = seq_warp_sum(d) * scale;
    const float mn = fmaxf(m, d);
    const float corr = expf(m - mn), pj = expf(d - mn);  // m = -inf on the first key: corr = 0
    l = l * corr + pj;
#pragma unroll
    for (int i = 0; i < kLatMaxPerLane; ++i) {
      const int c = lane + 32 * i;
      if (c < r) acc[i] = acc[i] * corr + pj * ldf(kr + c);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kLatMaxPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < r) sacc[warp * r + c] = acc[i];
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  float mt = -INFINITY;
#pragma unroll
  for (int w = 0; w < kLatWarps; ++w) mt = fmaxf(mt, s_m[w]);
  if (sink != nullptr) mt = fmaxf(mt, sink[h]);
  float lt = sink != nullptr ? expf(sink[h] - mt) : 0.f;
  float f[kLatWarps];
#pragma unroll
  for (int w = 0; w < kLatWarps; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - mt);
    lt += s_l[w] * f[w];
  }
  const float inv = 1.f / lt;
  float* o = out + ((long long)t * H + h) * r;
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) v += sacc[w * r + c] * f[w];
    o[c] = v * inv;
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_latent_kv_store(const float* dkv, long long ld, int T, int r, int dr, const void* w, int w_dt, float eps,
                                   const float* cs, int rot_dims, const int32_t* pos, const int32_t* slot,
                                   const int32_t* block_table, int max_pages, int page_size, void* pool, int pool_dt, void* stream) {
  if (dkv == nullptr || w == nullptr || cs == nullptr || pos == nullptr || slot == nullptr || block_table == nullptr || pool == nullptr ||
      T < 0 || r <= 0 || dr < 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1) || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_latent_kv_store: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(pool_dt, TC, {
    latent_kv_store_kernel<TW, TC><<<T, 128, 0, st>>>(dkv, ld, r, dr, static_cast<const TW*>(w), eps, cs, rot_dims, pos, slot,
                                                      block_table, max_pages, page_size, static_cast<TC*>(pool));
  }))
  return check_launch("omc_latent_kv_store");
}

extern "C" int omc_rotary_q(const float* q32, long long ldq, int T, int H, int dn, int dr, const float* cs, int rot_dims,
                            const int32_t* pos, void* qcat, int q_dt, int r, void* stream) {
  if (q32 == nullptr || cs == nullptr || pos == nullptr || qcat == nullptr || T < 0 || H <= 0 || dn < 0 || dr < 0 || rot_dims > dr ||
      (rot_dims & 1))
    return set_error(OMC_ERR_ARG, "omc_rotary_q: bad argument");
  if (T == 0 || dr == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(q_dt, TQ, { rotary_q_kernel<TQ><<<T, 128, 0, st>>>(q32, ldq, H, dn, dr, cs, rot_dims, pos, static_cast<TQ*>(qcat), r); })
  return check_launch("omc_rotary_q");
}

extern "C" int omc_latent_attn(const void* qcat, int q_dt, int T, int H, int r, int dr, const void* pool, int pool_dt,
                               const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot,
                               const float* sink, float scale, float* out, void* stream) {
  if (qcat == nullptr || pool == nullptr || block_table == nullptr || pos == nullptr || slot == nullptr || out == nullptr || T < 0 ||
      H <= 0 || r <= 0 || dr < 0 || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_latent_attn: bad argument");
  if (r > 32 * kLatMaxPerLane) return set_error(OMC_ERR_SHAPE, "omc_latent_attn: latent width above 1024");
  if (H > 65535) return set_error(OMC_ERR_SHAPE, "omc_latent_attn: more than 65535 heads");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(float) * ((size_t)r + dr + (size_t)kLatWarps * r + 2 * kLatWarps);
  OMC_DT_SWITCH(q_dt, TQ, OMC_DT_SWITCH(pool_dt, TC, {
    latent_attn_kernel<TQ, TC><<<dim3(T, H), kLatWarps * 32, smem, st>>>(static_cast<const TQ*>(qcat), H, r, dr,
                                                                         static_cast<const TC*>(pool), block_table, max_pages,
                                                                         page_size, pos, slot, sink, scale, out);
  }))
  return check_launch("omc_latent_attn");
}
