// Row kernels of decoders whose residual stream is fp32: scaled embedding gather, RMS norm of fp32 rows, and the
// output-side norm + residual add (x <- x + y / rms(y) * (1 + g)) that also emits the rounded copy the next sublayer reads.
// One CTA per row; the row is read once into registers / shared memory, the statistics are fp32. HBM-bound row work.
#include "seq_common.cuh"

namespace omc {

template <typename TT, typename TB>
__global__ void __launch_bounds__(256) embed_scale_kernel(const int32_t* __restrict__ ids, const TT* __restrict__ table, int C,
                                                          int vocab, float scale, float* __restrict__ h32, long long ldh,
                                                          TB* __restrict__ xb, long long ldxb) {
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = ok ? ldf(table + (long long)id * C + c) * scale : 0.f;
    h32[(long long)t * ldh + c] = v;
    if (xb != nullptr) stf(xb + (long long)t * ldxb + c, v);
  }
}

template <typename TW, typename TY>
__global__ void __launch_bounds__(256) rms_rows_kernel(const float* __restrict__ x, long long ldx, const TW* __restrict__ w,
                                                       int one_plus, float eps, TY* __restrict__ y, long long ldy, int n) {
  __shared__ float red[33];
  const float* xr = x + (long long)blockIdx.x * ldx;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float g = 1.f;
    if (w != nullptr) g = one_plus ? 1.f + ldf(w + c) : ldf(w + c);
    stf(y + (long long)blockIdx.x * ldy + c, xr[c] * rstd * g);
  }
}

template <typename TW, typename TB>
__global__ void __launch_bounds__(256) norm_residual_kernel(const float* __restrict__ y, long long ldy, const TW* __restrict__ w,
                                                            float eps, float* __restrict__ h32, long long ldh,
                                                            TB* __restrict__ xb, long long ldxb, int C) {
  __shared__ float red[33];
  const float* yr = y + (long long)blockIdx.x * ldy;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = yr[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = h32[(long long)blockIdx.x * ldh + c] + yr[c] * rstd * (1.f + ldf(w + c));
    h32[(long long)blockIdx.x * ldh + c] = v;
    if (xb != nullptr) stf(xb + (long long)blockIdx.x * ldxb + c, v);
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_embed_scale(const int32_t* ids, int T, const void* table, int t_dt, int C, int vocab, float scale, float* h32,
                               long long ldh, void* xb, int xb_dt, long long ldxb, void* stream) {
  if (ids == nullptr || table == nullptr || h32 == nullptr || T < 0 || C <= 0) return set_error(OMC_ERR_ARG, "omc_embed_scale: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(t_dt, TT, OMC_DT_SWITCH(xb_dt, TB, {
    embed_scale_kernel<TT, TB><<<T, 256, 0, st>>>(ids, static_cast<const TT*>(table), C, vocab, scale, h32, ldh,
                                                   static_cast<TB*>(xb), ldxb);
  }))
  return check_launch("omc_embed_scale");
}

extern "C" int omc_rms_rows(const float* x, long long ldx, const void* w, int w_dt, int one_plus, float eps, void* y, int y_dt,
                            long long ldy, int rows, int n, void* stream) {
  if (x == nullptr || y == nullptr || rows < 0 || n <= 0) return set_error(OMC_ERR_ARG, "omc_rms_rows: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(y_dt, TY, {
    rms_rows_kernel<TW, TY><<<rows, 256, 0, st>>>(x, ldx, static_cast<const TW*>(w), one_plus, eps, static_cast<TY*>(y), ldy, n);
  }))
  return check_launch("omc_rms_rows");
}

extern "C" int omc_norm_residual(const float* y, long long ldy, const void* w, int w_dt, float eps, float* h32, long long ldh,
                                 void* xb, int xb_dt, long long ldxb, int rows, int C, void* stream) {
  if (y == nullptr || w == nullptr || h32 == nullptr || rows < 0 || C <= 0) return set_error(OMC_ERR_ARG, "omc_norm_residual: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(xb_dt, TB, {
    norm_residual_kernel<TW, TB><<<rows, 256, 0, st>>>(y, ldy, static_cast<const TW*>(w), eps, h32, ldh, static_cast<TB*>(xb), ldxb, C);
  }))
  return check_launch("omc_norm_residual");
}
