// Pieces around the mixers of a post-norm decoder: the embedding with a sinusoidal position vector added, the
// residual update x += scale * RMSNorm(y) with a one-number norm weight and a per-feature layer scale, and the
// RMSNorm of a whole q or k projection (one statistic per token over all heads) with the store into the pages.
// Every statistic, angle and sum is float32 (the angle's product and its reduction to one turn are float64).
// These kernels take every size.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------
// out[n, 2i] = table[id, 2i] + sin(a), out[n, 2i+1] = table[id, 2i+1] + cos(a), a = position[n] * inv_freq[i].
// inv_freq is float64 (base^(-2i/width), made once on the host); the product is reduced to (-pi, pi] in float64
// before the float32 sine and cosine, so that a position in the hundreds of thousands loses nothing.
// half (may be null): the same row rounded to bfloat16, for the products that read the stream.
// An id outside the vocabulary reads nothing: the row is the position vector alone and the error word is set.
// ------------------------------------------------------------------------------------------
__global__ void embed_sinusoid_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                                      const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                      float* __restrict__ out, __nv_bfloat16* __restrict__ half, int hidden, int vocab,
                                      int* __restrict__ err) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  const int id = ids[n];
  const bool bad = id < 0 || id >= vocab;
  if (bad && err && threadIdx.x == 0) atomicCAS(err, 0, IFB_DEV_ERR_TOKEN_ID);
  const size_t row = bad ? 0 : (size_t)id * hidden;
  const double p = (double)positions[n];
  const double two_pi = 6.283185307179586476925286766559;
  for (int i = threadIdx.x; 2 * i < hidden; i += blockDim.x) {
    double a = p * inv_freq[i];
    a -= two_pi * rint(a / two_pi);
    float s, c;
    sincosf((float)a, &s, &c);
    const int e0 = 2 * i, e1 = 2 * i + 1;
    const float v0 = (bad ? 0.f : load_as_f32(table, table_dtype, row + e0)) + s;
    out[(size_t)n * hidden + e0] = v0;
    if (half) half[(size_t)n * hidden + e0] = __float2bfloat16_rn(v0);
    if (e1 < hidden) {
      const float v1 = (bad ? 0.f : load_as_f32(table, table_dtype, row + e1)) + c;
      out[(size_t)n * hidden + e1] = v1;
      if (half) half[(size_t)n * hidden + e1] = __float2bfloat16_rn(v1);
    }
  }
}

IFB_EXPORT int ifb_embed_sinusoid(const void* table, int table_dtype, const int* ids, const int* positions,
                                  const double* inv_freq, float* out, void* half, int n, int hidden, int vocab, int* err,
                                  cudaStream_t stream) {
  if (n <= 0 || hidden <= 0) return IFB_OK;
  if (table_dtype != IFB_F32 && table_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  const int pairs = (hidden + 1) / 2;
  const int threads = pairs >= 256 ? 256 : ((pairs + 31) / 32) * 32;
  return ifb_launch(embed_sinusoid_kernel, dim3(n), dim3(threads), 0, stream, table, table_dtype, ids, positions, inv_freq,
                    out, (__nv_bfloat16*)half, hidden, vocab, err);
}

// ------------------------------------------------------------------------------------------
// x[n, :] += y[n, :] / sqrt(mean(y[n, :]^2) + eps) * g * scale[:]      (g: one number; scale: per feature)
// half (may be null): the updated row rounded to bfloat16.  A block per row; a row of up to 8 * 256 * 4 features stays
// in registers between the two passes, a longer one is read twice.
// ------------------------------------------------------------------------------------------
constexpr int RP_THREADS = 256, RP_KEEP = 8;
__global__ void __launch_bounds__(RP_THREADS)
residual_postnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const void* __restrict__ g, int g_dtype,
                         const void* __restrict__ scale, int scale_dtype, float eps, __nv_bfloat16* __restrict__ half,
                         int hidden) {
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const size_t base = (size_t)blockIdx.x * hidden;
  const float* yr = y + base;
  float keep[RP_KEEP];
  float ss = 0.f;
  const bool held = hidden <= RP_KEEP * RP_THREADS;
  if (held) {
#pragma unroll
    for (int j = 0; j < RP_KEEP; ++j) {
      const int e = threadIdx.x + j * RP_THREADS;
      keep[j] = e < hidden ? yr[e] : 0.f;
      ss += keep[j] * keep[j];
    }
  } else {
    for (int e = threadIdx.x; e < hidden; e += RP_THREADS) { const float v = yr[e]; ss += v * v; }
  }
  ss = block_sum(ss, scratch);
  const float r = load_as_f32(g, g_dtype, 0) / sqrtf(ss / (float)hidden + eps);
  if (held) {
#pragma unroll
    for (int j = 0; j < RP_KEEP; ++j) {
      const int e = threadIdx.x + j * RP_THREADS;
      if (e < hidden) {
        const float v = x[base + e] + keep[j] * r * load_as_f32(scale, scale_dtype, e);
        x[base + e] = v;
        if (half) half[base + e] = __float2bfloat16_rn(v);
      }
    }
  } else {
    for (int e = threadIdx.x; e < hidden; e += RP_THREADS) {
      const float v = x[base + e] + yr[e] * r * load_as_f32(scale, scale_dtype, e);
      x[base + e] = v;
      if (half) half[base + e] = __float2bfloat16_rn(v);
    }
  }
}

IFB_EXPORT int ifb_residual_postnorm(float* x, const float* y, const void* g, int g_dtype, const void* scale, int scale_dtype,
                                     float eps, void* half, int n, int hidden, cudaStream_t stream) {
  if (n <= 0 || hidden <= 0) return IFB_OK;
  if ((g_dtype != IFB_F32 && g_dtype != IFB_BF16) || (scale_dtype != IFB_F32 && scale_dtype != IFB_BF16)) return IFB_ERR_DTYPE;
  return ifb_launch(residual_postnorm_kernel, dim3(n), dim3(RP_THREADS), 0, stream, x, y, g, g_dtype, scale, scale_dtype, eps,
                    (__nv_bfloat16*)half, hidden);
}

// out = x rounded to bfloat16, element by element.
__global__ void cast_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long count) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(x[i]);
}

IFB_EXPORT int ifb_cast_rows(const float* x, void* out, long long count, cudaStream_t stream) {
  if (count <= 0) return IFB_OK;
  const long long blocks = (count + 255) / 256;
  return ifb_launch(cast_rows_kernel, dim3((unsigned)(blocks > 4096 ? 4096 : blocks)), dim3(256), 0, stream, x,
                    (__nv_bfloat16*)out, count);
}

// ------------------------------------------------------------------------------------------
// The q and k projections of a token, each normalised as ONE vector over all its heads:
//   q_out[n, :]  = q / sqrt(mean(q^2) + eps) * qw        (q: proj[n, 0 : q_width])
//   key page     = k / sqrt(mean(k^2) + eps) * kw        (k: proj[n, q_width : q_width + k_width])
//   value page   = k before its norm (values_are_keys), or proj[n, v_col : v_col + k_width]
// written at slot = page * page_size + offset of pages [pages][2][kv_heads][page_size][head_dim]; a negative slot
// stores nothing.  A null weight leaves that projection unnormalised.  proj is float32; T is the cache's type.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
wide_norm_store_kernel(const float* __restrict__ proj, int ld, int q_width, int k_width, int v_col, int head_dim,
                       const void* __restrict__ qw, const void* __restrict__ kw, int w_dtype, float eps,
                       T* __restrict__ q_out, const int* __restrict__ slots, T* __restrict__ pages, int page_size) {
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int n = blockIdx.x;
  const float* row = proj + (size_t)n * ld;
  float sq = 0.f, sk = 0.f;
  if (qw) for (int e = threadIdx.x; e < q_width; e += blockDim.x) { const float v = row[e]; sq += v * v; }
  if (kw) for (int e = threadIdx.x; e < k_width; e += blockDim.x) { const float v = row[q_width + e]; sk += v * v; }
  const float rq = qw ? 1.f / sqrtf(block_sum(sq, scratch) / (float)q_width + eps) : 1.f;
  const float rk = kw ? 1.f / sqrtf(block_sum(sk, scratch) / (float)k_width + eps) : 1.f;
  for (int e = threadIdx.x; e < q_width; e += blockDim.x)
    q_out[(size_t)n * q_width + e] = from_f32<T>(qw ? row[e] * rq * load_as_f32(qw, w_dtype, e) : row[e]);
  const int slot = slots ? slots[n] : -1;
  if (slot < 0) return;
  const int kv_heads = k_width / head_dim;
  const size_t head_stride = (size_t)page_size * head_dim;
  T* kp = pages + (size_t)(slot / page_size) * 2 * kv_heads * head_stride + (size_t)(slot % page_size) * head_dim;
  T* vp = kp + (size_t)kv_heads * head_stride;
  for (int e = threadIdx.x; e < k_width; e += blockDim.x) {
    const int g = e / head_dim, d = e % head_dim;
    const float k = row[q_width + e];
    kp[(size_t)g * head_stride + d] = from_f32<T>(kw ? k * rk * load_as_f32(kw, w_dtype, e) : k);
    vp[(size_t)g * head_stride + d] = from_f32<T>(v_col < 0 ? k : row[v_col + e]);
  }
}

IFB_EXPORT int ifb_wide_norm_store(const float* proj, int ld, int q_width, int k_width, int v_col, int head_dim, const void* qw,
                                   const void* kw, int w_dtype, float eps, void* q_out, int out_dtype, const int* slots,
                                   void* pages, int page_size, int n, cudaStream_t stream) {
  if (n <= 0) return IFB_OK;
  if (head_dim < 1 || k_width % head_dim || q_width % head_dim || page_size < 1) return IFB_ERR_ARG;
  if (w_dtype != IFB_F32 && w_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (out_dtype == IFB_F32)
    return ifb_launch(wide_norm_store_kernel<float>, dim3(n), dim3(256), 0, stream, proj, ld, q_width, k_width, v_col, head_dim,
                      qw, kw, w_dtype, eps, (float*)q_out, slots, (float*)pages, page_size);
  if (out_dtype == IFB_BF16)
    return ifb_launch(wide_norm_store_kernel<__nv_bfloat16>, dim3(n), dim3(256), 0, stream, proj, ld, q_width, k_width, v_col,
                      head_dim, qw, kw, w_dtype, eps, (__nv_bfloat16*)q_out, slots, (__nv_bfloat16*)pages, page_size);
  return IFB_ERR_DTYPE;
}
