// Softmax attention over the paged cache in which the heads' scores are mixed before the softmax, with a linear
// distance bias and an optional chunk rule, in plain float32 arithmetic.  It serves every way a step can be cut
// (prompts, portions, single decoded tokens, mixed) and every size; q, the pages and the output may be float32 or
// bfloat16, and all arithmetic between loading and storing is float32.
//
// For the query at position p of a request, the keys first .. p are visible, first = (p / chunk) * chunk with a chunk
// rule, else 0.  With H query heads, head j reading key/value head j / (H / G):
//     a[j][s] = scale * q_j . k_g(s) - slope_j * (p - s),     slope_j = 2^(-slope_exp * (j + 1) / H)   (0: no bias)
//     b[j][s] = sum_i talk[j][i] * a[i][s]                                                          (null: b = a)
//     o_j     = sum_s softmax_s(b[j][:]) v_g(s)
//     out_j   = o_j * sigmoid(gate_j)                                                          (null gate: out = o)
// Because b needs every head's score of a (query, key) pair, a block is one query token with all its heads.  Keys are
// taken 32 at a time: a warp per head scores them (a lane per key), the block mixes the heads through shared memory,
// and a warp per head carries that head's running maximum, sum and output row.
#include "common.cuh"
#include <math.h>

struct TalkArgs {
  const void* q;            // [tokens][H * d], T
  const void* pages;        // [pages][2][G][page_size][d], T
  const int* block_tables;
  int bt_stride;
  const int* cu_q;
  const int* seq_lens;
  const void* talk;         // [H][H] or null
  int talk_dtype;
  const float* gate;        // row n at gate + n * gate_ld, H * d numbers before the sigmoid; or null
  int gate_ld;
  void* out;                // [tokens][H * d], T
  int n_tokens, n_req, H, G, d, page_size, chunk;
  float scale, slope_exp;
};

constexpr int TK_KEYS = 32;

template <typename T>
__global__ void __launch_bounds__(256)
attention_talk_kernel(TalkArgs a) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int tok = blockIdx.x;
  const int H = a.H, d = a.d;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* orow = (T*)a.out + (size_t)tok * H * d;
  int lo = 0, hi = a.n_req;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.cu_q[mid] <= tok) lo = mid; else hi = mid; }
  const int r = lo;
  const int q_len = a.cu_q[r + 1] - a.cu_q[r];
  const int p = tok < a.cu_q[a.n_req] ? a.seq_lens[r] - q_len + (tok - a.cu_q[r]) : -1;
  if (p < 0) {                                            // padding: no request stands behind this row
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) orow[i] = from_f32<T>(0.f);
    return;
  }
  float* qs = sm;                         // [H][d]
  float* acc = qs + H * d;                // [H][d]
  float* raw = acc + H * d;               // [H][32]
  float* mixed = raw + H * TK_KEYS;       // [H][32]
  float* tk = mixed + H * TK_KEYS;        // [H][H]
  float* ms = tk + H * H;                 // [H] running maximum
  float* ls = ms + H;                     // [H] running sum
  const T* qp = (const T*)a.q + (size_t)tok * H * d;
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) { qs[i] = to_f32<T>(qp[i]); acc[i] = 0.f; }
  if (a.talk) for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = load_as_f32(a.talk, a.talk_dtype, i);
  for (int i = threadIdx.x; i < H; i += blockDim.x) { ms[i] = -INFINITY; ls[i] = 0.f; }
  __syncthreads();
  const int first = a.chunk > 0 ? (p / a.chunk) * a.chunk : 0;
  const int* bt = a.block_tables + (size_t)r * a.bt_stride;
  const int rep = H / a.G;
  const size_t head_stride = (size_t)a.page_size * d, page_stride = 2 * (size_t)a.G * head_stride;
  const T* pages = (const T*)a.pages;
  for (int k0 = first; k0 <= p; k0 += TK_KEYS) {
    const int key = k0 + lane;
    const bool valid = key <= p;
    const T* kbase = nullptr;
    if (valid) kbase = pages + (size_t)bt[key / a.page_size] * page_stride + (size_t)(key % a.page_size) * d;
    for (int h = warp; h < H; h += warps) {               // scores of 32 keys for head h
      float s = 0.f;
      if (valid) {
        const T* kp = kbase + (size_t)(h / rep) * head_stride;
        const float* qh = qs + h * d;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(qh[i], to_f32<T>(kp[i]), dot);
        const float slope = a.slope_exp > 0.f ? exp2f(-a.slope_exp * (float)(h + 1) / (float)H) : 0.f;
        s = dot * a.scale - slope * (float)(p - key);
      }
      raw[h * TK_KEYS + lane] = s;
    }
    __syncthreads();
    if (a.talk) {
      for (int idx = threadIdx.x; idx < H * TK_KEYS; idx += blockDim.x) {
        const int h = idx / TK_KEYS, j = idx % TK_KEYS;
        float s = 0.f;
        for (int g = 0; g < H; ++g) s = fmaf(tk[h * H + g], raw[g * TK_KEYS + j], s);
        mixed[idx] = s;
      }
      __syncthreads();
    }
    const float* sc = a.talk ? mixed : raw;
    const int count = min(TK_KEYS, p - k0 + 1);
    for (int h = warp; h < H; h += warps) {               // softmax step and weighted sum of values for head h
      const float s = valid ? sc[h * TK_KEYS + lane] : -INFINITY;
      const float m_old = ms[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float pj = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m_old - m_new);             // exp(-inf) = 0 on the first tile
      const float l_new = ls[h] * corr + warp_sum(pj);
      __syncwarp();
      if (lane == 0) { ms[h] = m_new; ls[h] = l_new; }
      float* ah = acc + h * d;
      for (int i = lane; i < d; i += 32) ah[i] *= corr;
      const size_t voff = ((size_t)a.G + h / rep) * head_stride;
      for (int j = 0; j < count; ++j) {
        const float pv = __shfl_sync(0xffffffffu, pj, j);
        const int kj = k0 + j;
        const T* vp = pages + (size_t)bt[kj / a.page_size] * page_stride + voff + (size_t)(kj % a.page_size) * d;
        for (int i = lane; i < d; i += 32) ah[i] = fmaf(pv, to_f32<T>(vp[i]), ah[i]);
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
    float o = acc[i] / ls[i / d];
    if (a.gate) o *= 1.f / (1.f + expf(-a.gate[(size_t)tok * a.gate_ld + i]));
    orow[i] = from_f32<T>(o);
  }
}

IFB_EXPORT int ifb_attention_talk(const void* q, int dtype, const void* pages, const int* block_tables, int bt_stride,
                                  const int* cu_q, const int* seq_lens, const void* talk, int talk_dtype, const float* gate,
                                  int gate_ld, void* out, int n_tokens, int n_req, int H, int G, int d, int page_size, int chunk,
                                  float scale, float slope_exp, cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (H < 1 || G < 1 || H % G || d < 1 || page_size < 1 || chunk < 0) return IFB_ERR_ARG;
  if (talk && talk_dtype != IFB_F32 && talk_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  TalkArgs a{q, pages, block_tables, bt_stride, cu_q, seq_lens, talk, talk_dtype, gate, gate_ld, out, n_tokens, n_req, H, G, d,
             page_size, chunk, scale, slope_exp};
  const size_t smem = ((size_t)2 * H * d + 2 * H * TK_KEYS + (size_t)H * H + 2 * H) * sizeof(float);
  if (smem > 200 * 1024) return IFB_ERR_SIZE;
  if (dtype == IFB_F32) {
    IFB_ALLOW_SMEM(attention_talk_kernel<float>, smem);
    return ifb_launch(attention_talk_kernel<float>, dim3(n_tokens), dim3(256), smem, stream, a);
  }
  if (dtype == IFB_BF16) {
    IFB_ALLOW_SMEM(attention_talk_kernel<__nv_bfloat16>, smem);
    return ifb_launch(attention_talk_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), smem, stream, a);
  }
  return IFB_ERR_DTYPE;
}
