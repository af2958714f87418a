// The gated linear recurrence of an HGRN2 mixer, for prompts, portions of prompts and single decoded tokens alike.
//
// Per request and head a float32 state S [dim][vdim] lives in the request's state slot.  For each of the request's
// tokens of this step, in order:
//     q = silu(q_raw),  f = lower + (1 - lower) * sigmoid(f_raw + bias)                       (dim numbers each)
//     S[i][c] = f[i] * S[i][c] + (1 - f[i]) * v[c]
//     o[c]    = sum_i S[i][c] * q[i]
//     out[c]  = o[c] / sqrt(mean_c(o^2) + eps) * norm_weight[c]
// The columns c of S evolve independently, so a thread owns one column with its dim entries in registers; a block is
// one (request, head) with a thread per column.  Tokens are staged in groups: the block loads q_raw, f_raw and v of a
// group into shared memory and applies the activations once per number while doing so, every thread then walks the
// group's tokens, and at the end of the group the head's outputs are normalised, a warp per token.  A head with more
// columns than a block has threads (the more rows a thread keeps, the fewer threads a block may have) is split into
// slabs of columns, a block each; the outputs then go to a float32 scratch and a second kernel normalises them.
// Everything is float32; proj holds the projections as the product wrote them (float32).
//
// Long portions are cut into blocks of GS_BLOCK tokens that run side by side, in three launches: (A) every block is
// walked from a zero state, which leaves its own contribution Z_b and the product A_b of its gates (per row); (B) a
// thread per state element carries the state over the blocks, S_(b+1) = A_b * S_b + Z_b, leaving in Z_b's place the
// state S_b at the block's start, and writes the request's final state to its slot; (C) every block is walked again
// from S_b, now writing outputs.  Twice the arithmetic of the one-launch walk, for (tokens / GS_BLOCK) times as many
// blocks in flight.  The result differs from the one-launch walk by rounding only (the recurrence is linear in S).
#include "common.cuh"
#include <math.h>

constexpr int GS_GROUP = 16;       // tokens staged at a time

struct GatedScanArgs {
  const float* proj;       // [tokens][ld]: q_raw at q_col, f_raw at f_col (heads * dim each), v at v_col (heads * vdim)
  int ld, q_col, f_col, v_col;
  const void* bias;        // [heads * dim]
  const void* lower;       // [heads * dim]
  const void* norm_w;      // [vdim], shared by the heads
  int w_dtype;
  float eps;
  float* state;            // [slots][heads][dim][vdim]
  const int* state_slots;  // [requests]
  const int* cu_q;         // [requests + 1]
  const int* seq_lens;     // [requests]; a request of length 0 is padding and is skipped
  void* out;               // [tokens][heads * vdim], T
  float* raw;              // [tokens][heads * vdim]: the outputs before the norm, when a head has several slabs (else null)
  int heads, dim, vdim, slabs;
  int mode;                // 0: a request per block row, from and to its slot.  1: launch A.  2: launch C.
  int requests;
  float* z;                // [blocks][heads][dim][vdim]: launch A writes Z_b, launch B turns it into S_b, launch C reads it
  float* decay;            // [blocks][heads][dim]: A_b
};

constexpr int GS_BLOCK = 64;       // tokens of a block of the three-launch form (a multiple of GS_GROUP)

// The block of GS_BLOCK tokens that a CTA row is: request, first and last token.  False: the row is beyond the last block.
__device__ __forceinline__ bool gs_find_block(const GatedScanArgs& a, int row, int& r, int& t0, int& t1) {
  for (int i = 0; i < a.requests; ++i) {
    const int ql = a.seq_lens[i] > 0 ? a.cu_q[i + 1] - a.cu_q[i] : 0;
    const int blocks = (ql + GS_BLOCK - 1) / GS_BLOCK;
    if (row < blocks) {
      r = i;
      t0 = a.cu_q[i] + row * GS_BLOCK;
      t1 = min(a.cu_q[i + 1], t0 + GS_BLOCK);
      return true;
    }
    row -= blocks;
  }
  return false;
}

constexpr int gs_max_threads(int dmax) { return dmax <= 32 ? 512 : dmax <= 64 ? 256 : 128; }

// OUT false (launch A only): the walk leaves no outputs, so the sums S^T q are not formed.
template <typename T, int DMAX, bool OUT>
__global__ void __launch_bounds__(gs_max_threads(DMAX), 1)
gated_scan_kernel(GatedScanArgs a) {
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
  } else if (!gs_find_block(a, blockIdx.y, r, t0, t1)) {
    return;
  }
  float* qs = sm;                              // [GROUP][DMAX]
  float* fs = qs + GS_GROUP * DMAX;            // [GROUP][DMAX]
  float* vs = fs + GS_GROUP * DMAX;            // [GROUP][threads]
  float* os = vs + GS_GROUP * blockDim.x;      // [GROUP][threads]
  const bool col = c < vdim;
  // where the walk starts from and where its last state goes
  float* sp = a.mode == 0 ? a.state + (((size_t)a.state_slots[r] * a.heads + h) * dim) * vdim + c
                          : a.z + (((size_t)blockIdx.y * a.heads + h) * dim) * vdim + c;
  float* ap = os + GS_GROUP * blockDim.x;       // [DMAX]: launch A, the product of the block's gates
  if (a.mode == 1) for (int i = threadIdx.x; i < DMAX; i += blockDim.x) ap[i] = 1.f;
  float S[DMAX];
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (a.mode != 1 && col && i < dim) ? sp[(size_t)i * vdim] : 0.f;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // With rows of 33 to 64 (the usual head) a block of at least 128 threads asks for the next group's numbers while it
  // walks the present one: the walk is a chain per thread, and with few warps on an SM nothing else hides the loads.
  constexpr bool AHEAD = DMAX == 64;
  constexpr int QF = AHEAD ? GS_GROUP * DMAX / 128 : 1;
  float nq[QF], nf[QF], nv[AHEAD ? GS_GROUP : 1];
  const bool ahead = AHEAD && blockDim.x >= 128;
  auto fetch = [&](int g0) {
    const int cnt = min(GS_GROUP, t1 - g0);
#pragma unroll
    for (int j = 0; j < QF; ++j) {
      const int idx = threadIdx.x + j * blockDim.x, t = idx / DMAX, i = idx % DMAX;
      nq[j] = nf[j] = 0.f;
      if (idx < cnt * DMAX && i < dim) {
        const float* row = a.proj + (size_t)(g0 + t) * a.ld;
        nq[j] = row[a.q_col + h * dim + i];
        nf[j] = row[a.f_col + h * dim + i];
      }
    }
#pragma unroll
    for (int t = 0; t < (AHEAD ? GS_GROUP : 1); ++t)
      nv[t] = (t < cnt && col) ? a.proj[(size_t)(g0 + t) * a.ld + a.v_col + h * vdim + c] : 0.f;
  };
  if (ahead) fetch(t0);
  for (int g0 = t0; g0 < t1; g0 += GS_GROUP) {
    const int cnt = min(GS_GROUP, t1 - g0);
    // rows dim .. DMAX-1 are padding: f = 1 keeps their (zero) entries, q = 0 keeps them out of the sums
    if (ahead) {
#pragma unroll
      for (int j = 0; j < QF; ++j) {
        const int idx = threadIdx.x + j * blockDim.x, i = idx % DMAX;
        if (idx >= cnt * DMAX) continue;
        float qv = 0.f, fv = 1.f;
        if (i < dim) {
          qv = nq[j] / (1.f + expf(-nq[j]));
          const float lo = load_as_f32(a.lower, a.w_dtype, h * dim + i);
          const float z = nf[j] + load_as_f32(a.bias, a.w_dtype, h * dim + i);
          fv = lo + (1.f - lo) * (1.f / (1.f + expf(-z)));
        }
        qs[idx] = qv;
        fs[idx] = fv;
      }
#pragma unroll
      for (int t = 0; t < (AHEAD ? GS_GROUP : 1); ++t)
        if (t < cnt) vs[t * blockDim.x + threadIdx.x] = nv[t];
    } else {
      for (int idx = threadIdx.x; idx < cnt * DMAX; idx += blockDim.x) {
        const int t = idx / DMAX, i = idx % DMAX;
        float qv = 0.f, fv = 1.f;
        if (i < dim) {
          const float* row = a.proj + (size_t)(g0 + t) * a.ld;
          const float qr = row[a.q_col + h * dim + i];
          qv = qr / (1.f + expf(-qr));
          const float lo = load_as_f32(a.lower, a.w_dtype, h * dim + i);
          const float z = row[a.f_col + h * dim + i] + load_as_f32(a.bias, a.w_dtype, h * dim + i);
          fv = lo + (1.f - lo) * (1.f / (1.f + expf(-z)));
        }
        qs[idx] = qv;
        fs[idx] = fv;
      }
      for (int idx = threadIdx.x; idx < cnt * width; idx += blockDim.x) {
        const int t = idx / width, e = idx % width;
        vs[t * blockDim.x + e] = a.proj[(size_t)(g0 + t) * a.ld + a.v_col + h * vdim + c0 + e];
      }
    }
    __syncthreads();
    if (ahead && g0 + GS_GROUP < t1) fetch(g0 + GS_GROUP);
    if (a.mode == 1)                            // each row's gates of this group into the block's product (a row has one owner)
      for (int i = threadIdx.x; i < DMAX; i += blockDim.x) {
        float pr = ap[i];
        for (int t = 0; t < cnt; ++t) pr *= fs[t * DMAX + i];
        ap[i] = pr;
      }
    if (col) {
      for (int t = 0; t < cnt; ++t) {
        const float v = vs[t * blockDim.x + threadIdx.x];
        const float4* q = reinterpret_cast<const float4*>(qs + t * DMAX);
        const float4* f = reinterpret_cast<const float4*>(fs + t * DMAX);
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < DMAX / 4; ++i) {
          const float4 fi = f[i];
          S[4 * i] = fmaf(fi.x, S[4 * i], (1.f - fi.x) * v);
          S[4 * i + 1] = fmaf(fi.y, S[4 * i + 1], (1.f - fi.y) * v);
          S[4 * i + 2] = fmaf(fi.z, S[4 * i + 2], (1.f - fi.z) * v);
          S[4 * i + 3] = fmaf(fi.w, S[4 * i + 3], (1.f - fi.w) * v);
          if (OUT) {
            const float4 qi = q[i];
            o0 = fmaf(S[4 * i], qi.x, o0); o1 = fmaf(S[4 * i + 1], qi.y, o1);
            o2 = fmaf(S[4 * i + 2], qi.z, o2); o3 = fmaf(S[4 * i + 3], qi.w, o3);
          }
        }
        os[t * blockDim.x + threadIdx.x] = (o0 + o1) + (o2 + o3);
      }
    }
    __syncthreads();
    for (int t = warp; t < cnt && a.mode != 1; t += warps) {           // the head's norm, a warp per token
      const float* o = os + t * blockDim.x;
      if (a.raw) {                                      // the head has other slabs: its norm is the second kernel's
        float* dst = a.raw + ((size_t)(g0 + t) * a.heads + h) * vdim + c0;
        for (int e = lane; e < width; e += 32) dst[e] = o[e];
        continue;
      }
      float ss = 0.f;
      for (int e = lane; e < vdim; e += 32) ss += o[e] * o[e];
      const float rn = 1.f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
      T* dst = (T*)a.out + ((size_t)(g0 + t) * a.heads + h) * vdim;
      for (int e = lane; e < vdim; e += 32) dst[e] = from_f32<T>(o[e] * rn * load_as_f32(a.norm_w, a.w_dtype, e));
    }
    __syncthreads();
  }
  if (col && a.mode != 2) {
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
      if (i < dim) sp[(size_t)i * vdim] = S[i];
  }
  if (a.mode == 1 && c0 == 0)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) a.decay[((size_t)blockIdx.y * a.heads + h) * dim + i] = ap[i];
}

// Launch B: a thread per element (head, row, column) of a request's state carries it over the request's blocks.
__global__ void __launch_bounds__(256)
gated_scan_carry_kernel(GatedScanArgs a) {
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
    first += (ql + GS_BLOCK - 1) / GS_BLOCK;
  }
  const int blocks = (a.cu_q[r + 1] - a.cu_q[r] + GS_BLOCK - 1) / GS_BLOCK;
  const size_t hi = e / a.vdim;                    // (head, row): the gate's index
  float* slot = a.state + (size_t)a.state_slots[r] * per + e;
  float S = *slot;
  // eight blocks at a time: their loads are all asked for before the chain of multiply-adds that needs them
  for (int b0 = 0; b0 < blocks; b0 += 8) {
    float z[8], g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = b0 + j < blocks;
      z[j] = in ? __ldcg(a.z + (size_t)(first + b0 + j) * per + e) : 0.f;
      g[j] = in ? __ldg(a.decay + (size_t)(first + b0 + j) * a.heads * a.dim + hi) : 1.f;
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
// columns; per token the activated q and f of the head go through shared memory, every thread updates its columns row
// by row, and the block normalises the head's output.  Slow (the state crosses the memory bus for every token) and
// exact; no model met so far has such heads.
template <typename T>
__global__ void __launch_bounds__(256)
gated_scan_wide_kernel(GatedScanArgs a) {
  extern __shared__ float sm[];
  __shared__ float scratch[33];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int r = blockIdx.y, h = blockIdx.x, dim = a.dim, vdim = a.vdim;
  if (a.seq_lens[r] <= 0) return;
  float* qs = sm;              // [dim]
  float* fs = sm + dim;        // [dim]
  float* os = fs + dim;        // [vdim]
  float* S = a.state + ((size_t)a.state_slots[r] * a.heads + h) * dim * vdim;
  for (int t = a.cu_q[r]; t < a.cu_q[r + 1]; ++t) {
    const float* row = a.proj + (size_t)t * a.ld;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      const float qr = row[a.q_col + h * dim + i];
      qs[i] = qr / (1.f + expf(-qr));
      const float lo = load_as_f32(a.lower, a.w_dtype, h * dim + i);
      const float z = row[a.f_col + h * dim + i] + load_as_f32(a.bias, a.w_dtype, h * dim + i);
      fs[i] = lo + (1.f - lo) * (1.f / (1.f + expf(-z)));
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
      const float v = row[a.v_col + h * vdim + c];
      float o = 0.f;
      for (int i = 0; i < dim; ++i) {
        const float sv = fmaf(fs[i], S[(size_t)i * vdim + c], (1.f - fs[i]) * v);
        S[(size_t)i * vdim + c] = sv;
        o = fmaf(sv, qs[i], o);
      }
      os[c] = o;
      ss += o * o;
    }
    ss = block_sum(ss, scratch);
    const float rn = 1.f / sqrtf(ss / (float)vdim + a.eps);
    T* dst = (T*)a.out + ((size_t)t * a.heads + h) * vdim;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) dst[c] = from_f32<T>(os[c] * rn * load_as_f32(a.norm_w, a.w_dtype, c));
    __syncthreads();
  }
}

// out[t, h, :] = raw[t, h, :] / sqrt(mean(raw[t, h, :]^2) + eps) * w, a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kernel(const float* __restrict__ raw, const void* __restrict__ w, int w_dtype, float eps, T* __restrict__ out,
                 long long items, int vdim) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const float* o = raw + item * vdim;
  float ss = 0.f;
  for (int e = lane; e < vdim; e += 32) ss += o[e] * o[e];
  const float rn = 1.f / sqrtf(warp_sum(ss) / (float)vdim + eps);
  for (int e = lane; e < vdim; e += 32) out[item * vdim + e] = from_f32<T>(o[e] * rn * load_as_f32(w, w_dtype, e));
}

static int gs_block_threads(int dim, int vdim) {
  const int cap = gs_max_threads(dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : 128);
  return min(cap, ((vdim + 31) / 32) * 32);
}

template <typename T>
static int gs_launch(GatedScanArgs a, int requests, int tokens, cudaStream_t s) {
  if (a.dim > 128) {
    const size_t wide = (size_t)(2 * a.dim + a.vdim) * sizeof(float);
    if (wide > 200 * 1024) return IFB_ERR_SIZE;
    IFB_ALLOW_SMEM(gated_scan_wide_kernel<T>, wide);
    return ifb_launch(gated_scan_wide_kernel<T>, dim3(a.heads, requests), dim3(256), wide, s, a);
  }
  const int threads = gs_block_threads(a.dim, a.vdim);
  a.slabs = (a.vdim + threads - 1) / threads;
  if (a.slabs > 1 && !a.raw) return IFB_ERR_ARG;
  if (a.slabs == 1) a.raw = nullptr;
  dim3 grid(a.heads * a.slabs, a.mode == 0 ? requests : (tokens + GS_BLOCK - 1) / GS_BLOCK + requests);
  int st = IFB_ERR_SIZE;
  bool done = false;
#define GS_CASE(D)                                                                     \
  if (!done && a.dim <= D) {                                                           \
    const size_t smem = ((size_t)GS_GROUP * (2 * D + 2 * threads) + D) * sizeof(float); \
    done = true;                                                                       \
    if (a.mode == 1) {                                                                 \
      IFB_ALLOW_SMEM((gated_scan_kernel<T, D, false>), smem);                          \
      st = ifb_launch(gated_scan_kernel<T, D, false>, grid, dim3(threads), smem, s, a); \
    } else {                                                                           \
      IFB_ALLOW_SMEM((gated_scan_kernel<T, D, true>), smem);                           \
      st = ifb_launch(gated_scan_kernel<T, D, true>, grid, dim3(threads), smem, s, a); \
    }                                                                                  \
  }
  GS_CASE(16) GS_CASE(32) GS_CASE(64) GS_CASE(128)
#undef GS_CASE
  if (st != IFB_OK || a.slabs == 1 || a.mode == 1) return st;
  const long long items = (long long)tokens * a.heads;
  return ifb_launch(head_norm_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, (const float*)a.raw, a.norm_w,
                    a.w_dtype, a.eps, (T*)a.out, items, a.vdim);
}

// Slabs of columns that a head of these sizes is split into; with more than one the caller gives `raw`.
IFB_EXPORT int ifb_gated_scan_slabs(int dim, int vdim) {
  if (dim > 128) return 1;
  const int threads = gs_block_threads(dim, vdim);
  return (vdim + threads - 1) / threads;
}

// Floats of scratch (z, then decay) that the three-launch form needs for a step of these sizes.
IFB_EXPORT long long ifb_gated_scan_scratch_floats(int tokens, int requests, int heads, int dim, int vdim) {
  const long long blocks = (tokens + GS_BLOCK - 1) / GS_BLOCK + requests;
  return blocks * heads * dim * ((long long)vdim + 1);
}

template <typename T>
static int gs_run(GatedScanArgs a, int requests, int tokens, float* scratch, cudaStream_t s) {
  if (!scratch || a.dim > 128) return gs_launch<T>(a, requests, tokens, s);
  const long long blocks = (tokens + GS_BLOCK - 1) / GS_BLOCK + requests;
  a.z = scratch;
  a.decay = scratch + blocks * a.heads * a.dim * (long long)a.vdim;
  a.mode = 1;
  int st = gs_launch<T>(a, requests, tokens, s);
  if (st != IFB_OK) return st;
  const size_t per = (size_t)a.heads * a.dim * a.vdim;
  st = ifb_launch(gated_scan_carry_kernel, dim3((unsigned)((per + 255) / 256), requests), dim3(256), 0, s, a);
  if (st != IFB_OK) return st;
  a.mode = 2;
  return gs_launch<T>(a, requests, tokens, s);
}

// Any dim and vdim (dim over 128: the slow kernel with the state in device memory).  bias, lower and norm_w share one dtype.  raw: float32 [tokens][heads * vdim] scratch, needed
// when ifb_gated_scan_slabs(dim, vdim) > 1.  scratch: null for the one-launch walk (a request per block row); else
// ifb_gated_scan_scratch_floats(...) floats for the three-launch form, in which blocks of 64 tokens run side by side.
IFB_EXPORT int ifb_gated_scan(const float* proj, int ld, int q_col, int f_col, int v_col, const void* bias, const void* lower,
                              const void* norm_w, int w_dtype, float eps, float* state, const int* state_slots, const int* cu_q,
                              const int* seq_lens, void* out, int out_dtype, float* raw, float* scratch, int requests, int tokens,
                              int heads, int dim, int vdim, cudaStream_t stream) {
  if (requests <= 0 || tokens <= 0) return IFB_OK;
  if (heads < 1 || dim < 1 || vdim < 1 || requests > 65535) return IFB_ERR_SIZE;
  if (w_dtype != IFB_F32 && w_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  GatedScanArgs a{proj, ld, q_col, f_col, v_col, bias, lower, norm_w, w_dtype, eps, state, state_slots, cu_q, seq_lens, out,
                  raw, heads, dim, vdim, 1, 0, requests, nullptr, nullptr};
  if (out_dtype == IFB_F32) return gs_run<float>(a, requests, tokens, scratch, stream);
  if (out_dtype == IFB_BF16) return gs_run<__nv_bfloat16>(a, requests, tokens, scratch, stream);
  return IFB_ERR_DTYPE;
}
