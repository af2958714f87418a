// Linear recurrences over a request's state slot, for prompts, portions of prompts and single decoded tokens alike.
//
// (1) A matrix state per head.  Per request and head a float32 state S [dim][vdim] lives in the request's slot.  For
// each of the request's tokens of this step, in order, with a decay d[i] per row, a key k[i], a query q[i] and a value
// v[c]:
//     plain form         S[i][c] = d[i] S[i][c] + k[i] v[c];   o[c] = sum_i S[i][c] q[i]
//     with a bonus u[i]  o[c] = sum_i (S[i][c] + u[i] k[i] v[c]) q[i];   then S[i][c] = d[i] S[i][c] + k[i] v[c]
// (the output is read BEFORE the update and the token's own k v^T enters it through the bonus only).  The decay is
// either one constant per head (retention) or exp(-exp(w[i] + bias[i])) from a raw per-token row (RWKV-style time
// mixing); keys are multiplied by key_scale.  Then out[c] = o[c] / sqrt(mean_c(o^2) + eps) (* norm_w[head][c])
// (* silu(gate[c])).  The sum with the bonus splits into sum_i S[i][c] q[i] + v[c] * (sum_i u[i] k[i] q[i]); the
// second factor is one number per token and head, formed when the token is staged.
//
// The columns c of S evolve independently, so a thread owns one column with its dim entries in registers; a block is
// one (request, head) with a thread per column; tokens are staged in groups through shared memory, where decay, scaled
// key and the bonus number are formed once per token.  Rows dim .. DMAX-1 of the register tile are padding (decay 1,
// key 0, query 0).  A head with more columns than a block has threads is split into slabs of columns, a block each; the
// outputs then go to a float32 scratch and a second kernel finishes them.  Heads of more than 128 rows run a slow
// kernel with the state in device memory.
//
// Long portions are cut into blocks of LS_BLOCK tokens that run side by side, in three launches: (A) every block is
// walked from a zero state, which leaves its own contribution Z_b and the product A_b of its decays per row; (B) a
// thread per state element carries the state over the blocks, S_(b+1) = A_b S_b + Z_b, leaving S_b in Z_b's place and
// the final state in the slot; (C) every block is walked again from S_b, now writing outputs.  The result differs
// from the one-launch walk by rounding only (the recurrence is linear in S).
//
// (2) An element-wise gated unit (minGRU): S[c] = (1 - z[c]) S[c] + z[c] cand[c] per element of a state [width],
// a thread per (request, element).
//
// Everything is float32; the inputs are the projections as their products wrote them (float32).
#include "common.cuh"
#include <math.h>

constexpr int LS_GROUP = 16;       // tokens staged at a time
constexpr int LS_BLOCK = 64;       // tokens of a block of the three-launch form (a multiple of LS_GROUP)

struct LinearScanArgs {
  const float *q, *k, *v, *w, *gate;     // rows [tokens][ld]; head h at columns h * dim (q, k, w) or h * vdim (v, gate)
  int ldq, ldk, ldv, ldw, ldg;           // w: the raw decay (null with a constant decay); gate may be null
  const float* decay;                    // [heads]: the constant decay of each head, or null
  const void* w_bias;                    // [heads * dim]: added to w before exp(-exp(.)), when decay is null
  const void* bonus;                     // [heads * dim] or null
  const void* norm_w;                    // [heads * vdim] or null
  int p_dtype;                           // dtype of w_bias, bonus and norm_w
  float key_scale, eps;
  float* state;                          // [slots][heads][dim][vdim]
  const int* state_slots;                // [requests]
  const int* cu_q;                       // [requests + 1]
  const int* seq_lens;                   // [requests]; a request of length 0 is padding and is skipped
  void* out;                             // [tokens][heads * vdim], T
  float* raw;                            // [tokens][heads * vdim]: outputs before the finish, when a head has several slabs
  int heads, dim, vdim, slabs;
  int mode;                              // 0: a request per block row, from and to its slot.  1: launch A.  2: launch C.
  int requests;
  float* z;                              // [blocks][heads][dim][vdim]
  float* dprod;                          // [blocks][heads][dim]
};

__device__ __forceinline__ bool ls_find_block(const LinearScanArgs& a, int row, int& r, int& t0, int& t1) {
  for (int i = 0; i < a.requests; ++i) {
    const int ql = a.seq_lens[i] > 0 ? a.cu_q[i + 1] - a.cu_q[i] : 0;
    const int blocks = (ql + LS_BLOCK - 1) / LS_BLOCK;
    if (row < blocks) {
      r = i;
      t0 = a.cu_q[i] + row * LS_BLOCK;
      t1 = min(a.cu_q[i + 1], t0 + LS_BLOCK);
      return true;
    }
    row -= blocks;
  }
  return false;
}

constexpr int ls_max_threads(int dmax) { return dmax <= 32 ? 512 : dmax <= 64 ? 256 : 128; }

// out = o / rms(o) (* norm_w) (* silu(gate)) for one (token, head), by one warp; the head's vdim sums are o[e], or with
// `parts` > 1 the sum over p of o[p * part_stride + e] (the rows of a column were split over several threads)
template <typename T>
__device__ __forceinline__ void ls_finish(const LinearScanArgs& a, const float* o, int t, int h, int lane, int parts = 1,
                                          int part_stride = 0) {
  const int vdim = a.vdim;
  float ss = 0.f;
  for (int e = lane; e < vdim; e += 32) {
    float v = o[e];
    for (int p = 1; p < parts; ++p) v += o[p * part_stride + e];
    ss += v * v;
  }
  const float rn = 1.f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
  T* dst = (T*)a.out + ((size_t)t * a.heads + h) * vdim;
  for (int e = lane; e < vdim; e += 32) {
    float v = o[e];
    for (int p = 1; p < parts; ++p) v += o[p * part_stride + e];
    float y = v * rn;
    if (a.norm_w) y *= load_as_f32(a.norm_w, a.p_dtype, (size_t)h * vdim + e);
    if (a.gate) { const float g = a.gate[(size_t)t * a.ldg + h * vdim + e]; y *= g / (1.f + expf(-g)); }
    dst[e] = from_f32<T>(y);
  }
}

// OUT false (launch A only): the walk leaves no outputs, so the sums S^T q are not formed.
template <typename T, int DMAX, bool OUT, bool BONUS>
__global__ void __launch_bounds__(ls_max_threads(DMAX), 1)
linear_scan_kernel(LinearScanArgs a) {
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int h = blockIdx.x / a.slabs, c0 = (blockIdx.x % a.slabs) * blockDim.x, c = c0 + threadIdx.x;
  const int dim = a.dim, vdim = a.vdim;
  const int width = min((int)blockDim.x, vdim - c0);        // columns of this block
  int r = blockIdx.y, t0, t1;
  if (a.mode == 0) {
    if (a.seq_lens[r] <= 0) return;
    t0 = a.cu_q[r]; t1 = a.cu_q[r + 1];
  } else if (!ls_find_block(a, blockIdx.y, r, t0, t1)) {
    return;
  }
  float* qs = sm;                              // [GROUP][DMAX]
  float* ks = qs + LS_GROUP * DMAX;            // [GROUP][DMAX]
  float* ds = ks + LS_GROUP * DMAX;            // [GROUP][DMAX]
  float* vs = ds + LS_GROUP * DMAX;            // [GROUP][threads]
  float* os = vs + LS_GROUP * blockDim.x;      // [GROUP][threads]
  float* ap = os + LS_GROUP * blockDim.x;      // [DMAX]: launch A, the product of the block's decays
  float* bs = ap + DMAX;                       // [GROUP]: the bonus number of each token
  const bool col = c < vdim;
  float* sp = a.mode == 0 ? a.state + (((size_t)a.state_slots[r] * a.heads + h) * dim) * vdim + c
                          : a.z + (((size_t)blockIdx.y * a.heads + h) * dim) * vdim + c;
  if (a.mode == 1) for (int i = threadIdx.x; i < DMAX; i += blockDim.x) ap[i] = 1.f;
  float S[DMAX];
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (a.mode != 1 && col && i < dim) ? sp[(size_t)i * vdim] : 0.f;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float head_decay = a.decay ? a.decay[h] : 1.f;
  for (int g0 = t0; g0 < t1; g0 += LS_GROUP) {
    const int cnt = min(LS_GROUP, t1 - g0);
    for (int idx = threadIdx.x; idx < cnt * DMAX; idx += blockDim.x) {
      const int t = idx / DMAX, i = idx % DMAX;
      float qv = 0.f, kv = 0.f, dv = 1.f;
      if (i < dim) {
        const size_t tok = (size_t)(g0 + t);
        qv = a.q[tok * a.ldq + h * dim + i];
        kv = a.k[tok * a.ldk + h * dim + i] * a.key_scale;
        dv = a.decay ? head_decay
                     : expf(-expf(a.w[tok * a.ldw + h * dim + i] + load_as_f32(a.w_bias, a.p_dtype, (size_t)h * dim + i)));
      }
      qs[idx] = qv;
      ks[idx] = kv;
      ds[idx] = dv;
    }
    for (int idx = threadIdx.x; idx < cnt * width; idx += blockDim.x) {
      const int t = idx / width, e = idx % width;
      vs[t * blockDim.x + e] = a.v[(size_t)(g0 + t) * a.ldv + h * vdim + c0 + e];
    }
    __syncthreads();
    if (BONUS)                                   // b_t = sum_i u[i] k[i] q[i], a warp per token
      for (int t = warp; t < cnt; t += warps) {
        float b = 0.f;
        for (int i = lane; i < dim; i += 32)
          b += load_as_f32(a.bonus, a.p_dtype, (size_t)h * dim + i) * ks[t * DMAX + i] * qs[t * DMAX + i];
        b = warp_sum(b);
        if (lane == 0) bs[t] = b;
      }
    if (a.mode == 1)                            // each row's decays of this group into the block's product (a row has one owner)
      for (int i = threadIdx.x; i < DMAX; i += blockDim.x) {
        float pr = ap[i];
        for (int t = 0; t < cnt; ++t) pr *= ds[t * DMAX + i];
        ap[i] = pr;
      }
    if (BONUS) __syncthreads();
    if (col) {
      for (int t = 0; t < cnt; ++t) {
        const float v = vs[t * blockDim.x + threadIdx.x];
        const float4* q4 = reinterpret_cast<const float4*>(qs + t * DMAX);
        const float4* k4 = reinterpret_cast<const float4*>(ks + t * DMAX);
        const float4* d4 = reinterpret_cast<const float4*>(ds + t * DMAX);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < DMAX / 4; ++i) {
          const float4 di = d4[i], ki = k4[i];
          if (OUT && BONUS) {                   // the output reads the state before this token's update
            const float4 qi = q4[i];
            o0 = fmaf(S[4 * i], qi.x, o0); o1 = fmaf(S[4 * i + 1], qi.y, o1);
            o2 = fmaf(S[4 * i + 2], qi.z, o2); o3 = fmaf(S[4 * i + 3], qi.w, o3);
          }
          S[4 * i] = fmaf(di.x, S[4 * i], ki.x * v);
          S[4 * i + 1] = fmaf(di.y, S[4 * i + 1], ki.y * v);
          S[4 * i + 2] = fmaf(di.z, S[4 * i + 2], ki.z * v);
          S[4 * i + 3] = fmaf(di.w, S[4 * i + 3], ki.w * v);
          if (OUT && !BONUS) {
            const float4 qi = q4[i];
            o0 = fmaf(S[4 * i], qi.x, o0); o1 = fmaf(S[4 * i + 1], qi.y, o1);
            o2 = fmaf(S[4 * i + 2], qi.z, o2); o3 = fmaf(S[4 * i + 3], qi.w, o3);
          }
        }
        float o = (o0 + o1) + (o2 + o3);
        if (OUT && BONUS) o = fmaf(v, bs[t], o);
        os[t * blockDim.x + threadIdx.x] = o;
      }
    }
    __syncthreads();
    for (int t = warp; t < cnt && a.mode != 1; t += warps) {           // the head's finish, a warp per token
      const float* o = os + t * blockDim.x;
      if (a.raw) {                                      // the head has other slabs: the second kernel finishes it
        float* dst = a.raw + ((size_t)(g0 + t) * a.heads + h) * vdim + c0;
        for (int e = lane; e < width; e += 32) dst[e] = o[e];
        continue;
      }
      ls_finish<T>(a, o, g0 + t, h, lane);
    }
    __syncthreads();
  }
  if (col && a.mode != 2) {
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
      if (i < dim) sp[(size_t)i * vdim] = S[i];
  }
  if (a.mode == 1 && c0 == 0)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) a.dprod[((size_t)blockIdx.y * a.heads + h) * dim + i] = ap[i];
}

// The same walk with the rows of a state column split over RS = 2 threads, each with DMAX / 2 of them in registers: a head
// of few columns then has twice the threads for staging its tokens (decay, key, bonus number), half the chain per thread
// and half the registers; the two partial sums of an output meet in shared memory at the finish.
template <typename T, int DMAX, int RS, bool OUT, bool BONUS>
__global__ void __launch_bounds__(ls_max_threads(DMAX), DMAX <= 64 ? 2 : 1)
linear_scan_split_kernel(LinearScanArgs a) {
  constexpr int RPT = DMAX / RS;               // rows per thread
  extern __shared__ float sm[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int cols = blockDim.x / RS;            // threads along the columns
  const int cid = threadIdx.x % cols, part = threadIdx.x / cols, r0 = part * RPT;
  const int h = blockIdx.x / a.slabs, c0 = (blockIdx.x % a.slabs) * cols, c = c0 + cid;
  const int dim = a.dim, vdim = a.vdim;
  const int width = min(cols, vdim - c0);      // columns of this block
  int r = blockIdx.y, t0, t1;
  if (a.mode == 0) {
    if (a.seq_lens[r] <= 0) return;
    t0 = a.cu_q[r]; t1 = a.cu_q[r + 1];
  } else if (!ls_find_block(a, blockIdx.y, r, t0, t1)) {
    return;
  }
  float* qs = sm;                              // [GROUP][DMAX]
  float* ks = qs + LS_GROUP * DMAX;            // [GROUP][DMAX]
  float* ds = ks + LS_GROUP * DMAX;            // [GROUP][DMAX]
  float* vs = ds + LS_GROUP * DMAX;            // [GROUP][cols]
  float* os = vs + LS_GROUP * cols;            // [RS][GROUP][cols]
  float* ap = os + RS * LS_GROUP * cols;       // [DMAX]: launch A, the product of the block's decays
  float* bs = ap + DMAX;                       // [GROUP]: the bonus number of each token
  const bool col = c < vdim;
  float* sp = a.mode == 0 ? a.state + (((size_t)a.state_slots[r] * a.heads + h) * dim) * vdim + c
                          : a.z + (((size_t)blockIdx.y * a.heads + h) * dim) * vdim + c;
  if (a.mode == 1) for (int i = threadIdx.x; i < DMAX; i += blockDim.x) ap[i] = 1.f;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) S[i] = (a.mode != 1 && col && r0 + i < dim) ? sp[(size_t)(r0 + i) * vdim] : 0.f;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float head_decay = a.decay ? a.decay[h] : 1.f;
  for (int g0 = t0; g0 < t1; g0 += LS_GROUP) {
    const int cnt = min(LS_GROUP, t1 - g0);
    for (int idx = threadIdx.x; idx < cnt * DMAX; idx += blockDim.x) {
      const int t = idx / DMAX, i = idx % DMAX;
      float qv = 0.f, kv = 0.f, dv = 1.f;
      if (i < dim) {
        const size_t tok = (size_t)(g0 + t);
        qv = a.q[tok * a.ldq + h * dim + i];
        kv = a.k[tok * a.ldk + h * dim + i] * a.key_scale;
        dv = a.decay ? head_decay
                     : expf(-expf(a.w[tok * a.ldw + h * dim + i] + load_as_f32(a.w_bias, a.p_dtype, (size_t)h * dim + i)));
      }
      qs[idx] = qv;
      ks[idx] = kv;
      ds[idx] = dv;
    }
    for (int idx = threadIdx.x; idx < cnt * width; idx += blockDim.x) {
      const int t = idx / width, e = idx % width;
      vs[t * cols + e] = a.v[(size_t)(g0 + t) * a.ldv + h * vdim + c0 + e];
    }
    __syncthreads();
    if (BONUS)                                   // b_t = sum_i u[i] k[i] q[i], a warp per token
      for (int t = warp; t < cnt; t += warps) {
        float b = 0.f;
        for (int i = lane; i < dim; i += 32)
          b += load_as_f32(a.bonus, a.p_dtype, (size_t)h * dim + i) * ks[t * DMAX + i] * qs[t * DMAX + i];
        b = warp_sum(b);
        if (lane == 0) bs[t] = b;
      }
    if (a.mode == 1)                            // each row's decays of this group into the block's product (a row has one owner)
      for (int i = threadIdx.x; i < DMAX; i += blockDim.x) {
        float pr = ap[i];
        for (int t = 0; t < cnt; ++t) pr *= ds[t * DMAX + i];
        ap[i] = pr;
      }
    if (BONUS) __syncthreads();
    if (col) {
      for (int t = 0; t < cnt; ++t) {
        const float v = vs[t * cols + cid];
        const float4* q4 = reinterpret_cast<const float4*>(qs + t * DMAX + r0);
        const float4* k4 = reinterpret_cast<const float4*>(ks + t * DMAX + r0);
        const float4* d4 = reinterpret_cast<const float4*>(ds + t * DMAX + r0);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 di = d4[i], ki = k4[i];
          if (OUT && BONUS) {                   // the output reads the state before this token's update
            const float4 qi = q4[i];
            o0 = fmaf(S[4 * i], qi.x, o0); o1 = fmaf(S[4 * i + 1], qi.y, o1);
            o2 = fmaf(S[4 * i + 2], qi.z, o2); o3 = fmaf(S[4 * i + 3], qi.w, o3);
          }
          S[4 * i] = fmaf(di.x, S[4 * i], ki.x * v);
          S[4 * i + 1] = fmaf(di.y, S[4 * i + 1], ki.y * v);
          S[4 * i + 2] = fmaf(di.z, S[4 * i + 2], ki.z * v);
          S[4 * i + 3] = fmaf(di.w, S[4 * i + 3], ki.w * v);
          if (OUT && !BONUS) {
            const float4 qi = q4[i];
            o0 = fmaf(S[4 * i], qi.x, o0); o1 = fmaf(S[4 * i + 1], qi.y, o1);
            o2 = fmaf(S[4 * i + 2], qi.z, o2); o3 = fmaf(S[4 * i + 3], qi.w, o3);
          }
        }
        float o = (o0 + o1) + (o2 + o3);
        if (OUT && BONUS && part == 0) o = fmaf(v, bs[t], o);
        os[(part * LS_GROUP + t) * cols + cid] = o;
      }
    }
    __syncthreads();
    for (int t = warp; t < cnt && a.mode != 1; t += warps) {           // the head's finish, a warp per token
      const float* o = os + t * cols;
      if (a.raw) {                                      // the head has other slabs: the second kernel finishes it
        float* dst = a.raw + ((size_t)(g0 + t) * a.heads + h) * vdim + c0;
        for (int e = lane; e < width; e += 32) {
          float v = o[e];
          for (int p = 1; p < RS; ++p) v += o[p * LS_GROUP * cols + e];
          dst[e] = v;
        }
        continue;
      }
      ls_finish<T>(a, o, g0 + t, h, lane, RS, LS_GROUP * cols);
    }
    __syncthreads();
  }
  if (col && a.mode != 2) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (r0 + i < dim) sp[(size_t)(r0 + i) * vdim] = S[i];
  }
  if (a.mode == 1 && c0 == 0)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) a.dprod[((size_t)blockIdx.y * a.heads + h) * dim + i] = ap[i];
}

// Launch B: a thread per element (head, row, column) of a request's state carries it over the request's blocks.
__global__ void __launch_bounds__(256)
linear_scan_carry_kernel(LinearScanArgs a) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y;
  if (a.seq_lens[r] <= 0) return;
  const size_t per = (size_t)a.heads * a.dim * a.vdim;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per) return;
  int first = 0;                                   // index of the request's first block among all blocks
  for (int i = 0; i < r; ++i) {
    const int ql = a.seq_lens[i] > 0 ? a.cu_q[i + 1] - a.cu_q[i] : 0;
    first += (ql + LS_BLOCK - 1) / LS_BLOCK;
  }
  const int blocks = (a.cu_q[r + 1] - a.cu_q[r] + LS_BLOCK - 1) / LS_BLOCK;
  const size_t hi = e / a.vdim;                    // (head, row): the decay's index
  float* slot = a.state + (size_t)a.state_slots[r] * per + e;
  float S = *slot;
  for (int b0 = 0; b0 < blocks; b0 += 8) {         // eight blocks' loads are asked for before the chain that needs them
    float z[8], g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = b0 + j < blocks;
      z[j] = in ? __ldcg(a.z + (size_t)(first + b0 + j) * per + e) : 0.f;
      g[j] = in ? __ldcg(a.dprod + (size_t)(first + b0 + j) * a.heads * a.dim + hi) : 1.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (b0 + j < blocks) a.z[(size_t)(first + b0 + j) * per + e] = S;
      S = fmaf(g[j], S, z[j]);
    }
  }
  *slot = S;
}

// Heads with more than 128 rows: the state stays in device memory.  A block per (request, head), its threads over the
// columns.  Slow (the state crosses the memory bus for every token) and exact.
template <typename T>
__global__ void __launch_bounds__(256)
linear_scan_wide_kernel(LinearScanArgs a) {
  extern __shared__ float sm[];
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y, h = blockIdx.x, dim = a.dim, vdim = a.vdim;
  if (a.seq_lens[r] <= 0) return;
  float* qs = sm;              // [dim]
  float* ks = qs + dim;        // [dim]
  float* ds = ks + dim;        // [dim]
  float* os = ds + dim;        // [vdim]
  float* S = a.state + ((size_t)a.state_slots[r] * a.heads + h) * dim * vdim;
  const int lane = threadIdx.x & 31;
  for (int t = a.cu_q[r]; t < a.cu_q[r + 1]; ++t) {
    float bpart = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      qs[i] = a.q[(size_t)t * a.ldq + h * dim + i];
      ks[i] = a.k[(size_t)t * a.ldk + h * dim + i] * a.key_scale;
      ds[i] = a.decay ? a.decay[h]
                      : expf(-expf(a.w[(size_t)t * a.ldw + h * dim + i] + load_as_f32(a.w_bias, a.p_dtype, (size_t)h * dim + i)));
      if (a.bonus) bpart += load_as_f32(a.bonus, a.p_dtype, (size_t)h * dim + i) * ks[i] * qs[i];
    }
    const float b = block_sum(bpart, scratch);       // also orders the staging before the walk
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
      const float v = a.v[(size_t)t * a.ldv + h * vdim + c];
      float o = 0.f;
      for (int i = 0; i < dim; ++i) {
        const float old = S[(size_t)i * vdim + c];
        const float sv = fmaf(ds[i], old, ks[i] * v);
        S[(size_t)i * vdim + c] = sv;
        o = fmaf(a.bonus ? old : sv, qs[i], o);
      }
      os[c] = a.bonus ? fmaf(v, b, o) : o;
    }
    __syncthreads();
    if (threadIdx.x < 32) ls_finish<T>(a, os, t, h, lane);
    __syncthreads();
  }
}

// The finish of heads that were walked in slabs: a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
linear_scan_finish_kernel(LinearScanArgs a, long long items) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int t = (int)(item / a.heads), h = (int)(item % a.heads);
  ls_finish<T>(a, a.raw + item * a.vdim, t, h, threadIdx.x & 31);
}

static int ls_block_threads(int dim, int vdim) {
  const int cap = ls_max_threads(dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : 128);
  return min(cap, ((vdim + 31) / 32) * 32);
}

// The rows of a column over two threads where the block then still fits (heads of more than 32 rows)
static int ls_row_split(int dim, int vdim) {
  const int cap = ls_max_threads(dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : 128);
  return (dim > 32 && 2 * ls_block_threads(dim, vdim) <= cap) ? 2 : 1;
}

template <typename T, bool BONUS>
static int ls_launch(LinearScanArgs a, int requests, int tokens, cudaStream_t s) {
  if (a.dim > 128) {
    const size_t wide = (size_t)(3 * a.dim + a.vdim) * sizeof(float);
    if (wide > 200 * 1024) return IFB_ERR_SIZE;
    IFB_ALLOW_SMEM(linear_scan_wide_kernel<T>, wide);
    return ifb_launch(linear_scan_wide_kernel<T>, dim3(a.heads, requests), dim3(256), wide, s, a);
  }
  const int threads = ls_block_threads(a.dim, a.vdim);          // threads along the columns
  const bool split = ls_row_split(a.dim, a.vdim) == 2;
  a.slabs = (a.vdim + threads - 1) / threads;
  if (a.slabs > 1 && !a.raw) return IFB_ERR_ARG;
  if (a.slabs == 1) a.raw = nullptr;
  dim3 grid(a.heads * a.slabs, a.mode == 0 ? requests : (tokens + LS_BLOCK - 1) / LS_BLOCK + requests);
  int st = IFB_ERR_SIZE;
  bool done = false;
#define LS_CASE(D)                                                                              \
  if (!done && a.dim <= D && !(split && D >= 64)) {                                             \
    const size_t smem = ((size_t)LS_GROUP * (3 * D + 2 * threads) + D + LS_GROUP) * sizeof(float); \
    done = true;                                                                                \
    if (a.mode == 1) {                                                                          \
      IFB_ALLOW_SMEM((linear_scan_kernel<T, D, false, BONUS>), smem);                           \
      st = ifb_launch(linear_scan_kernel<T, D, false, BONUS>, grid, dim3(threads), smem, s, a); \
    } else {                                                                                    \
      IFB_ALLOW_SMEM((linear_scan_kernel<T, D, true, BONUS>), smem);                            \
      st = ifb_launch(linear_scan_kernel<T, D, true, BONUS>, grid, dim3(threads), smem, s, a);  \
    }                                                                                           \
  }
#define LS_SPLIT(D)                                                                                       \
  if (!done && a.dim <= D && split) {                                                                     \
    const size_t smem = ((size_t)LS_GROUP * (3 * D + 3 * threads) + D + LS_GROUP) * sizeof(float);        \
    done = true;                                                                                          \
    if (a.mode == 1) {                                                                                    \
      IFB_ALLOW_SMEM((linear_scan_split_kernel<T, D, 2, false, BONUS>), smem);                            \
      st = ifb_launch(linear_scan_split_kernel<T, D, 2, false, BONUS>, grid, dim3(2 * threads), smem, s, a); \
    } else {                                                                                              \
      IFB_ALLOW_SMEM((linear_scan_split_kernel<T, D, 2, true, BONUS>), smem);                             \
      st = ifb_launch(linear_scan_split_kernel<T, D, 2, true, BONUS>, grid, dim3(2 * threads), smem, s, a);  \
    }                                                                                                     \
  }
  LS_CASE(16) LS_CASE(32) LS_SPLIT(64) LS_CASE(64) LS_SPLIT(128) LS_CASE(128)
#undef LS_CASE
#undef LS_SPLIT
  if (st != IFB_OK || a.slabs == 1 || a.mode == 1) return st;
  const long long items = (long long)tokens * a.heads;
  return ifb_launch(linear_scan_finish_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, a, items);
}

// Slabs of columns that a head of these sizes is split into; with more than one the caller gives `raw`.
IFB_EXPORT int ifb_linear_scan_slabs(int dim, int vdim) {
  if (dim > 128) return 1;
  const int threads = ls_block_threads(dim, vdim);
  return (vdim + threads - 1) / threads;
}

// Floats of scratch (z, then the decay products) that the three-launch form needs for a step of these sizes.
IFB_EXPORT long long ifb_linear_scan_scratch_floats(int tokens, int requests, int heads, int dim, int vdim) {
  const long long blocks = (tokens + LS_BLOCK - 1) / LS_BLOCK + requests;
  return blocks * heads * dim * ((long long)vdim + 1);
}

template <typename T, bool BONUS>
static int ls_run(LinearScanArgs a, int requests, int tokens, float* scratch, cudaStream_t s) {
  if (!scratch || a.dim > 128) return ls_launch<T, BONUS>(a, requests, tokens, s);
  const long long blocks = (tokens + LS_BLOCK - 1) / LS_BLOCK + requests;
  a.z = scratch;
  a.dprod = scratch + blocks * a.heads * a.dim * (long long)a.vdim;
  a.mode = 1;
  int st = ls_launch<T, BONUS>(a, requests, tokens, s);
  if (st != IFB_OK) return st;
  const size_t per = (size_t)a.heads * a.dim * a.vdim;
  st = ifb_launch(linear_scan_carry_kernel, dim3((unsigned)((per + 255) / 256), requests), dim3(256), 0, s, a);
  if (st != IFB_OK) return st;
  a.mode = 2;
  return ls_launch<T, BONUS>(a, requests, tokens, s);
}

// q, k, v, w, gate: float32 rows with their own leading dimensions.  Exactly one of decay (with w and w_bias null) and
// (w, w_bias) is given.  bonus, norm_w and gate may be null; w_bias, bonus and norm_w share one dtype.  raw: float32
// [tokens][heads * vdim] scratch, needed when ifb_linear_scan_slabs(dim, vdim) > 1.  scratch: null for the one-launch
// walk; else ifb_linear_scan_scratch_floats(...) floats for the three-launch form.
IFB_EXPORT int ifb_linear_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* w, int ldw,
                               const float* gate, int ldg, const float* decay, const void* w_bias, const void* bonus,
                               const void* norm_w, int p_dtype, float key_scale, float eps, float* state, const int* state_slots,
                               const int* cu_q, const int* seq_lens, void* out, int out_dtype, float* raw, float* scratch,
                               int requests, int tokens, int heads, int dim, int vdim, cudaStream_t stream) {
  if (requests <= 0 || tokens <= 0) return IFB_OK;
  if (heads < 1 || dim < 1 || vdim < 1 || requests > 65535) return IFB_ERR_SIZE;
  if (p_dtype != IFB_F32 && p_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if ((decay != nullptr) == (w != nullptr) || (w != nullptr) != (w_bias != nullptr)) return IFB_ERR_ARG;
  LinearScanArgs a{q, k, v, w, gate, ldq, ldk, ldv, ldw, ldg, decay, w_bias, bonus, norm_w, p_dtype, key_scale, eps, state,
                   state_slots, cu_q, seq_lens, out, raw, heads, dim, vdim, 1, 0, requests, nullptr, nullptr};
  if (out_dtype == IFB_F32)
    return bonus ? ls_run<float, true>(a, requests, tokens, scratch, stream) : ls_run<float, false>(a, requests, tokens, scratch, stream);
  if (out_dtype == IFB_BF16)
    return bonus ? ls_run<__nv_bfloat16, true>(a, requests, tokens, scratch, stream)
                 : ls_run<__nv_bfloat16, false>(a, requests, tokens, scratch, stream);
  return IFB_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------
// The gated unit.  proj [tokens][3 * width] holds z_raw | x_raw | g of every token.  Per request, in order:
//     z = sigmoid(z_raw + z_bias);  u = x_raw + x_bias;  cand = u >= 0 ? u + 1/2 : sigmoid(u)
//     S = (1 - z) S + z cand;   out = S * silu(g)
// A thread per (request, element); the loads of a token do not depend on the chain, so eight tokens' worth are asked
// for before the chain that needs them.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
gated_unit_scan_kernel(const float* __restrict__ proj, const void* __restrict__ z_bias, const void* __restrict__ x_bias,
                       int b_dtype, float* __restrict__ state, const int* __restrict__ state_slots,
                       const int* __restrict__ cu_q, const int* __restrict__ seq_lens, T* __restrict__ out, int width) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width || seq_lens[r] <= 0) return;
  const float bz = load_as_f32(z_bias, b_dtype, c), bx = load_as_f32(x_bias, b_dtype, c);
  float* sp = state + (size_t)state_slots[r] * width + c;
  float S = *sp;
  const int t1 = cu_q[r + 1];
  const size_t ld = 3 * (size_t)width;
  for (int t0 = cu_q[r]; t0 < t1; t0 += 8) {
    float zr[8], xr[8], gr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = t0 + j < t1;
      const float* row = proj + (size_t)(t0 + j) * ld;
      zr[j] = in ? row[c] : 0.f;
      xr[j] = in ? row[width + c] : 0.f;
      gr[j] = in ? row[2 * width + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (t0 + j >= t1) break;
      const float z = 1.f / (1.f + expf(-(zr[j] + bz)));
      const float u = xr[j] + bx;
      const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
      S = fmaf(z, cand - S, S);
      out[(size_t)(t0 + j) * width + c] = from_f32<T>(S * (gr[j] / (1.f + expf(-gr[j]))));
    }
  }
  *sp = S;
}

// Long portions of the gated unit, in chunks of GU_CHUNK tokens that run side by side, in two launches.  The recurrence
// is S = a S + b with a = 1 - z and b = z cand, so a chunk is the map S -> A S + B with A the product of its a and B its
// own end state from zero.  (A) every chunk forms (A, B); the request's first chunk also copies the slot's state aside.
// (B) every chunk folds the maps of the request's earlier chunks onto that copy, in order, walks its tokens from there and
// writes outputs; the request's last chunk writes the slot.  Differs from the one-launch walk by rounding only.
constexpr int GU_CHUNK = 64;

// The chunk that block row `row` is: request r, tokens t0 .. t1, its index j among the request's chunks, and the block row
// of the request's first chunk.  False: the row is beyond the last chunk.
__device__ __forceinline__ bool gu_find_chunk(const int* cu_q, const int* seq_lens, int requests, int row, int& r, int& t0, int& t1,
                                              int& j, int& first_row, bool& last) {
  int base = 0;
  for (int i = 0; i < requests; ++i) {
    const int ql = seq_lens[i] > 0 ? cu_q[i + 1] - cu_q[i] : 0;
    const int chunks = (ql + GU_CHUNK - 1) / GU_CHUNK;
    if (row - base < chunks) {
      r = i; j = row - base; first_row = base;
      t0 = cu_q[i] + j * GU_CHUNK;
      t1 = min(cu_q[i + 1], t0 + GU_CHUNK);
      last = j == chunks - 1;
      return true;
    }
    base += chunks;
  }
  return false;
}

template <typename T, bool WRITE>
__global__ void __launch_bounds__(128)
gated_unit_chunk_kernel(const float* __restrict__ proj, const void* __restrict__ z_bias, const void* __restrict__ x_bias,
                        int b_dtype, float* __restrict__ state, const int* __restrict__ state_slots,
                        const int* __restrict__ cu_q, const int* __restrict__ seq_lens, T* __restrict__ out, int width,
                        int requests, float* __restrict__ maps, float* __restrict__ init) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  int r, t0, t1, j, first_row;
  bool last;
  if (c >= width || !gu_find_chunk(cu_q, seq_lens, requests, blockIdx.y, r, t0, t1, j, first_row, last)) return;
  const float bz = load_as_f32(z_bias, b_dtype, c), bx = load_as_f32(x_bias, b_dtype, c);
  float* sp = state + (size_t)state_slots[r] * width + c;
  float S = 0.f, A = 1.f;
  if (WRITE) {
    S = init[(size_t)r * width + c];
    for (int i = 0; i < j; ++i) {
      const float2 m = *reinterpret_cast<const float2*>(maps + 2 * ((size_t)(first_row + i) * width + c));
      S = fmaf(m.x, S, m.y);
    }
  } else if (j == 0) {
    init[(size_t)r * width + c] = *sp;
  }
  const size_t ld = 3 * (size_t)width;
  for (int g0 = t0; g0 < t1; g0 += 8) {
    float zr[8], xr[8], gr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool in = g0 + i < t1;
      const float* row = proj + (size_t)(g0 + i) * ld;
      zr[i] = in ? row[c] : 0.f;
      xr[i] = in ? row[width + c] : 0.f;
      gr[i] = (in && WRITE) ? row[2 * width + c] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (g0 + i >= t1) break;
      const float z = 1.f / (1.f + expf(-(zr[i] + bz)));
      const float u = xr[i] + bx;
      const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
      S = fmaf(z, cand - S, S);
      if (WRITE) out[(size_t)(g0 + i) * width + c] = from_f32<T>(S * (gr[i] / (1.f + expf(-gr[i]))));
      else A *= 1.f - z;
    }
  }
  if (!WRITE) *reinterpret_cast<float2*>(maps + 2 * ((size_t)blockIdx.y * width + c)) = make_float2(A, S);
  else if (last) *sp = S;
}

// Floats of scratch that the chunked form needs.
IFB_EXPORT long long ifb_gated_unit_scratch_floats(int tokens, int requests, int width) {
  const long long rows = (tokens + GU_CHUNK - 1) / GU_CHUNK + requests;
  return (2 * rows + requests) * (long long)width;
}

template <typename T>
static int gu_chunked(const float* proj, const void* z_bias, const void* x_bias, int b_dtype, float* state, const int* state_slots,
                      const int* cu_q, const int* seq_lens, void* out, int requests, int tokens, int width, float* scratch,
                      cudaStream_t stream) {
  const int rows = (tokens + GU_CHUNK - 1) / GU_CHUNK + requests;
  if (rows > 65535) return IFB_ERR_SIZE;
  float* maps = scratch;
  float* init = scratch + 2 * (size_t)rows * width;
  dim3 grid((width + 127) / 128, rows);
  int st = ifb_launch(gated_unit_chunk_kernel<T, false>, grid, dim3(128), 0, stream, proj, z_bias, x_bias, b_dtype, state, state_slots,
                      cu_q, seq_lens, (T*)out, width, requests, maps, init);
  if (st != IFB_OK) return st;
  return ifb_launch(gated_unit_chunk_kernel<T, true>, grid, dim3(128), 0, stream, proj, z_bias, x_bias, b_dtype, state, state_slots,
                    cu_q, seq_lens, (T*)out, width, requests, maps, init);
}

IFB_EXPORT int ifb_gated_unit_scan(const float* proj, const void* z_bias, const void* x_bias, int b_dtype, float* state,
                                   const int* state_slots, const int* cu_q, const int* seq_lens, void* out, int out_dtype,
                                   int requests, int tokens, int width, float* scratch, cudaStream_t stream) {
  if (requests <= 0 || tokens <= 0 || width <= 0) return IFB_OK;
  if (requests > 65535) return IFB_ERR_SIZE;
  if (b_dtype != IFB_F32 && b_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  if (scratch) {          // ifb_gated_unit_scratch_floats(...) floats: the chunked form
    if (out_dtype == IFB_BF16)
      return gu_chunked<__nv_bfloat16>(proj, z_bias, x_bias, b_dtype, state, state_slots, cu_q, seq_lens, out, requests, tokens,
                                       width, scratch, stream);
    if (out_dtype != IFB_F32) return IFB_ERR_DTYPE;
    return gu_chunked<float>(proj, z_bias, x_bias, b_dtype, state, state_slots, cu_q, seq_lens, out, requests, tokens, width,
                             scratch, stream);
  }
  dim3 grid((width + 127) / 128, requests);
  if (out_dtype == IFB_BF16)
    return ifb_launch(gated_unit_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, proj, z_bias, x_bias, b_dtype, state,
                      state_slots, cu_q, seq_lens, (__nv_bfloat16*)out, width);
  if (out_dtype != IFB_F32) return IFB_ERR_DTYPE;
  return ifb_launch(gated_unit_scan_kernel<float>, grid, dim3(128), 0, stream, proj, z_bias, x_bias, b_dtype, state, state_slots,
                    cu_q, seq_lens, (float*)out, width);
}
