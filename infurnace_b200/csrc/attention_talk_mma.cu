// Attention with the heads' scores mixed before the softmax (see attention_talk.cu for the arithmetic), bfloat16
// operands on the tensor cores (mma.sync m16n8k16, float32 accumulation), for prompts, portions and decoded tokens.
//
// A CTA owns a tile of 16 query tokens of one request and a group of NW output heads, one per warp.  Keys of the
// tile's chunk are taken 32 at a time:
//   1. K and V of the group's key/value heads come into shared memory (16-byte async copies, asked for one tile ahead:
//      the keys while the tile before is mixed and consumed, the values while this tile's scores are formed and mixed);
//   2. warp w forms the raw scores of its head, S = Q K_g^T, scales them, subtracts the distance bias and leaves
//      them in shared memory in float32;
//   3. the block mixes: a thread forms b[o] = sum_h talk[o][h] * a[h] for four heads o of the group and four
//      neighbouring keys of one query, in float32 on the ordinary pipes (the scores are never rounded);
//   4. warp w carries head o = group * NW + w: running maximum and sum per row, P rounded to bfloat16 as the A
//      operand of O += P V, V read transposed from shared memory.
// The mixing needs every head's score of a (query, key) pair.  With more query heads than NW (16) the groups of one
// query tile are the CTAs of a thread-block cluster: each scores its own heads, and step 3 reads the other groups'
// scores out of their shared memory (mapa + ld.shared::cluster) between two cluster barriers, so that no score is
// formed twice and a CTA holds the queries, keys and values of its own heads only.  The output is multiplied by
// sigmoid(gate) and stored as bfloat16.  Head sizes 16, 32, 64, 128; up to 8 groups (128 heads).
// A step of few query tokens (decoding) has few tiles; its keys are then split over several CTAs per tile (each takes
// every splits-th tile of 32 keys; the mixing is per (query, key) pair, so any split of the keys is exact), and a
// second kernel merges the parts in a fixed order.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

struct TalkMmaArgs {
  const bf16* q;            // [tokens][H * D]
  const bf16* pages;        // [pages][2][G][page_size][D]
  const int* block_tables;
  int bt_stride;
  const int* cu_q;
  const int* seq_lens;
  const void* talk;         // [H][H] or null
  int talk_dtype;
  const float* gate;        // row n at gate + n * gate_ld; or null
  int gate_ld;
  bf16* out;                // [tokens][H * D]
  int n_tokens, n_req, H, G, page_size, chunk;
  float scale, slope_exp;
  int splits;               // > 1: CTA z takes every splits-th tile of keys and leaves its part in `parts` for the merge
  float* parts;             // [tokens][H][splits][D + 2]: the unnormalised output row, then the maximum and the sum
};

constexpr int TM_ROWS = 16, TM_KEYS = 32;

__device__ __forceinline__ uint32_t tm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(tm_smem(dst)), "l"(src));
}
__device__ __forceinline__ void tm_cp_wait() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void tm_cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void tm_cp_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }
__device__ __forceinline__ void tm_ldsm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(tm_smem(p)));
}
__device__ __forceinline__ void tm_ldsm4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(tm_smem(p)));
}
__device__ __forceinline__ void tm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t tm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// All threads of all CTAs of the cluster: arrive (release) and wait (acquire).  Every CTA of a cluster takes the same
// number of trips through the key loop (they share the query tile), and none leaves before the last barrier.
__device__ __forceinline__ void tm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Four floats at this CTA's shared address `addr`, read from the CTA of rank `rank` in the cluster.
__device__ __forceinline__ float4 tm_ld_cluster_f4(uint32_t addr, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// Shared memory, in this order: Q [NW][16][D + 8] bf16, K and V [GV][32][D + 8] bf16 each (GV: key/value heads of the
// group), S [NW][16][32] float, M [NW][16][32] float, talk^T [H][NW] float.  CL: the groups form a cluster.
template <int D, int NW, bool CL>
__global__ void __launch_bounds__(NW * 32, 1)
attention_talk_mma_kernel(TalkMmaArgs a, int gv_max) {
  extern __shared__ __align__(16) unsigned char tm_raw[];
  ifb_pdl_wait();
  ifb_pdl_trigger();
  constexpr int LD = D + 8;                               // row pitch in elements: 16-byte aligned, no bank conflicts
  const int H = a.H, G = a.G, rep = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  // which (request, tile) this CTA is
  int r = -1, tile = 0;
  {
    int left = blockIdx.x;
    for (int i = 0; i < a.n_req; ++i) {
      const int ql = a.seq_lens[i] > 0 ? a.cu_q[i + 1] - a.cu_q[i] : 0;     // a request of length 0 is padding
      const int tiles = (ql + TM_ROWS - 1) / TM_ROWS;
      if (left < tiles) { r = i; tile = left; break; }
      left -= tiles;
    }
  }
  if (r < 0) return;
  const int q_len = a.cu_q[r + 1] - a.cu_q[r];
  const int q0 = a.cu_q[r] + tile * TM_ROWS;
  const int rows = min(TM_ROWS, q_len - tile * TM_ROWS);
  const int p0 = a.seq_lens[r] - q_len + tile * TM_ROWS;            // position of the tile's first query
  const int p_last = p0 + rows - 1;
  const int o0 = blockIdx.y * NW;                                   // first head of the group
  const int heads_here = min(NW, H - o0);
  const int g_lo = o0 / rep, g_hi = (o0 + heads_here - 1) / rep, GV = g_hi - g_lo + 1;

  bf16* Qs = reinterpret_cast<bf16*>(tm_raw);
  bf16* Ks = Qs + (size_t)NW * TM_ROWS * LD;
  bf16* Vs = Ks + (size_t)gv_max * TM_KEYS * LD;
  float* Ss = reinterpret_cast<float*>(Vs + (size_t)gv_max * TM_KEYS * LD);
  float* Ms = Ss + (size_t)NW * TM_ROWS * TM_KEYS;
  float* Tt = Ms + (size_t)NW * TM_ROWS * TM_KEYS;                  // [H][NW]: talk[o0 + o][h] at Tt[h * NW + o]

  constexpr int CH = D / 8;                                         // 16-byte pieces of a head row
  for (int idx = tid; idx < heads_here * TM_ROWS * CH; idx += NW * 32) {
    const int c = idx % CH, i = (idx / CH) % TM_ROWS, h = idx / (CH * TM_ROWS);
    bf16* dst = Qs + ((size_t)h * TM_ROWS + i) * LD + c * 8;
    if (i < rows) tm_cp16(dst, a.q + (size_t)(q0 + i) * H * D + (size_t)(o0 + h) * D + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  if (a.talk)
    for (int idx = tid; idx < H * NW; idx += NW * 32) {
      const int h = idx / NW, o = idx % NW;
      Tt[idx] = o < heads_here ? load_as_f32(a.talk, a.talk_dtype, (size_t)(o0 + o) * H + h) : 0.f;
    }

  const int chunk = a.chunk;
  const int ps_shift = (a.page_size & (a.page_size - 1)) == 0 ? __ffs(a.page_size) - 1 : -1;
  const int first = chunk > 0 ? (p0 / chunk) * chunk : 0;           // the first key any row of the tile sees
  const int* bt = a.block_tables + (size_t)r * a.bt_stride;
  const size_t head_stride = (size_t)a.page_size * D, page_stride = 2 * (size_t)G * head_stride;
  const int rl = lane >> 2, cl = (lane & 3) * 2;                    // this lane's row and first column in an 8-wide tile
  const int pr0 = p0 + rl, pr1 = p0 + rl + 8;                       // positions of its two rows
  const int lo0 = chunk > 0 ? (pr0 / chunk) * chunk : 0, lo1 = chunk > 0 ? (pr1 / chunk) * chunk : 0;
  const bool row0 = rl < rows, row1 = rl + 8 < rows;

  float O[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // The copies of a tile's keys are asked for while the tile before it is mixed and consumed, those of its values while
  // its own scores are formed and mixed: K's buffer is free once the scores are out, V's once the tile is consumed.  Every
  // thread commits the same groups in the same order (K0 with the queries, V0, K1, V1, ...), so "all but the latest
  // group" is K of the present tile at the top of a trip and V of the present tile before its fourth step.
  auto load_tile = [&](int k0, bool is_v) {
    for (int idx = tid; idx < GV * TM_KEYS * CH; idx += NW * 32) {
      const int c = idx % CH, j = (idx / CH) % TM_KEYS, gg = idx / (CH * TM_KEYS);
      const int g = g_lo + gg;
      bf16* dst = (is_v ? Vs : Ks) + ((size_t)gg * TM_KEYS + j) * LD + c * 8;
      const int key = k0 + j;
      if (key <= p_last) {
        const int pi = ps_shift >= 0 ? key >> ps_shift : key / a.page_size;           // pages are nearly always 2^k tokens
        const int po = ps_shift >= 0 ? key & (a.page_size - 1) : key % a.page_size;
        const bf16* src = a.pages + (size_t)bt[pi] * page_stride + ((size_t)(is_v ? G : 0) + g) * head_stride +
                          (size_t)po * D + c * 8;
        tm_cp16(dst, src);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  const int k_first = first + (int)blockIdx.z * TM_KEYS, k_step = TM_KEYS * a.splits;
  if (k_first <= p_last) load_tile(k_first, false);
  tm_cp_commit();
  if (k_first <= p_last) load_tile(k_first, true);
  tm_cp_commit();
  for (int k0 = k_first; k0 <= p_last; k0 += k_step) {
    // ---- 1. this tile's keys have landed (its values may still be on their way)
    tm_cp_wait_but_one();
    __syncthreads();
    // ---- 2. raw scores of this warp's head
    if (warp < heads_here) {
      const int h = o0 + warp;
      float acc[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
      const bf16* qh = Qs + (size_t)warp * TM_ROWS * LD;
      const bf16* kg = Ks + (size_t)(h / rep - g_lo) * TM_KEYS * LD;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t af[4];
        tm_ldsm4(af, qh + (size_t)(lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {                 // two 8-key tiles per load
          uint32_t bfr[4];
          tm_ldsm4(bfr, kg + (size_t)(n2 * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
          tm_mma(acc[2 * n2], af, bfr[0], bfr[1]);
          tm_mma(acc[2 * n2 + 1], af, bfr[2], bfr[3]);
        }
      }
      const float slope = a.slope_exp > 0.f ? exp2f(-a.slope_exp * (float)(h + 1) / (float)H) : 0.f;
      float* sh = Ss + (size_t)warp * TM_ROWS * TM_KEYS;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n * 8 + cl, key = k0 + col;
        float2 v0 = make_float2(acc[n][0] * a.scale - slope * (float)(pr0 - key), acc[n][1] * a.scale - slope * (float)(pr0 - key - 1));
        float2 v1 = make_float2(acc[n][2] * a.scale - slope * (float)(pr1 - key), acc[n][3] * a.scale - slope * (float)(pr1 - key - 1));
        *reinterpret_cast<float2*>(sh + rl * TM_KEYS + col) = v0;
        *reinterpret_cast<float2*>(sh + (rl + 8) * TM_KEYS + col) = v1;
      }
    }
    if (CL) tm_cluster_sync(); else __syncthreads();      // every group's scores are in its shared memory
    if (k0 + k_step <= p_last) load_tile(k0 + k_step, false);      // K's buffer is free: the next tile's keys
    tm_cp_commit();
    // ---- 3. the heads' scores of each (query, key) pair mixed, for the group's heads
    const float* Sc = Ss;                                           // without mixing: the group's own scores
    if (a.talk) {
      // a thread takes four neighbouring keys of one query and four heads of the group: per source head one 16-byte
      // load of scores, one of weights (the same for the whole warp) and sixteen multiply-adds
      const int pq = tid & 127, oq = tid >> 7;            // 128 quads of pairs x NW / 4 quads of heads = the block
      float b[4][4];
#pragma unroll
      for (int o = 0; o < 4; ++o) { b[o][0] = b[o][1] = b[o][2] = b[o][3] = 0.f; }
      const uint32_t s_at = tm_smem(Ss) + (uint32_t)(pq * 16);
      // four source heads at a time: their scores (from a peer's shared memory, in a cluster) are asked for together
      for (int h0 = 0; h0 < H; h0 += 4) {
        float4 sv[4], tv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int h = min(h0 + u, H - 1);
          sv[u] = CL ? tm_ld_cluster_f4(s_at + (uint32_t)((h % NW) * TM_ROWS * TM_KEYS * 4), h / NW)
                     : *reinterpret_cast<const float4*>(Ss + (size_t)h * TM_ROWS * TM_KEYS + pq * 4);
          tv[u] = h0 + u < H ? *reinterpret_cast<const float4*>(Tt + h * NW + oq * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float4 s4 = sv[u], t4 = tv[u];
          b[0][0] = fmaf(t4.x, s4.x, b[0][0]); b[0][1] = fmaf(t4.x, s4.y, b[0][1]); b[0][2] = fmaf(t4.x, s4.z, b[0][2]); b[0][3] = fmaf(t4.x, s4.w, b[0][3]);
          b[1][0] = fmaf(t4.y, s4.x, b[1][0]); b[1][1] = fmaf(t4.y, s4.y, b[1][1]); b[1][2] = fmaf(t4.y, s4.z, b[1][2]); b[1][3] = fmaf(t4.y, s4.w, b[1][3]);
          b[2][0] = fmaf(t4.z, s4.x, b[2][0]); b[2][1] = fmaf(t4.z, s4.y, b[2][1]); b[2][2] = fmaf(t4.z, s4.z, b[2][2]); b[2][3] = fmaf(t4.z, s4.w, b[2][3]);
          b[3][0] = fmaf(t4.w, s4.x, b[3][0]); b[3][1] = fmaf(t4.w, s4.y, b[3][1]); b[3][2] = fmaf(t4.w, s4.z, b[3][2]); b[3][3] = fmaf(t4.w, s4.w, b[3][3]);
        }
      }
#pragma unroll
      for (int o = 0; o < 4; ++o)
        *reinterpret_cast<float4*>(Ms + (size_t)(oq * 4 + o) * TM_ROWS * TM_KEYS + pq * 4) = make_float4(b[o][0], b[o][1], b[o][2], b[o][3]);
      Sc = Ms;
    }
    tm_cp_wait_but_one();                                 // this tile's values have landed (the next keys may be on their way)
    // the mixed scores are in place; and nobody writes its scores of the next tile while a peer still reads these
    if (CL) tm_cluster_sync(); else __syncthreads();
    // ---- 4. softmax step and O += P V for this warp's head
    if (warp < heads_here) {
      const float* sw = Sc + (size_t)warp * TM_ROWS * TM_KEYS;
      float s[4][4];
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n * 8 + cl, key = k0 + col;
        const float2 v0 = *reinterpret_cast<const float2*>(sw + rl * TM_KEYS + col);
        const float2 v1 = *reinterpret_cast<const float2*>(sw + (rl + 8) * TM_KEYS + col);
        s[n][0] = (row0 && key >= lo0 && key <= pr0) ? v0.x : -INFINITY;
        s[n][1] = (row0 && key + 1 >= lo0 && key + 1 <= pr0) ? v0.y : -INFINITY;
        s[n][2] = (row1 && key >= lo1 && key <= pr1) ? v1.x : -INFINITY;
        s[n][3] = (row1 && key + 1 >= lo1 && key + 1 <= pr1) ? v1.y : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;     // a row that has seen no key yet
      const float c0 = __expf(m0 - b0), c1 = __expf(m1 - b1);      // P is rounded to bfloat16 below: ex2's error is far under that
      m0 = n0; m1 = n1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pa[2][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const float e0 = __expf(s[n][0] - b0), e1 = __expf(s[n][1] - b0), e2 = __expf(s[n][2] - b1), e3 = __expf(s[n][3] - b1);
        sum0 += e0 + e1; sum1 += e2 + e3;
        pa[n >> 1][(n & 1) * 2] = tm_pack(e0, e1);
        pa[n >> 1][(n & 1) * 2 + 1] = tm_pack(e2, e3);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * c0 + sum0; l1 = l1 * c1 + sum1;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) { O[n][0] *= c0; O[n][1] *= c0; O[n][2] *= c1; O[n][3] *= c1; }
      const bf16* vg = Vs + (size_t)((o0 + warp) / rep - g_lo) * TM_KEYS * LD;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < D / 16; ++n2) {            // two 8-wide tiles of the head per load
          uint32_t bfr[4];
          tm_ldsm4_t(bfr, vg + (size_t)(kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + n2 * 16 + (lane >> 4) * 8);
          tm_mma(O[2 * n2], pa[kk], bfr[0], bfr[1]);
          tm_mma(O[2 * n2 + 1], pa[kk], bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();
    if (k0 + k_step <= p_last) load_tile(k0 + k_step, true);       // V's buffer is free: the next tile's values
    tm_cp_commit();
  }
  tm_cp_wait();                             // a CTA without a tile of keys has the copies of its queries in flight
  if (warp >= heads_here) return;
  const int head = o0 + warp;
  if (a.splits > 1) {                       // this CTA's part: rows as they are, with their maxima and sums
    float* pr0p = a.parts + (((size_t)(q0 + rl) * H + head) * a.splits + blockIdx.z) * (D + 2);
    float* pr1p = a.parts + (((size_t)(q0 + rl + 8) * H + head) * a.splits + blockIdx.z) * (D + 2);
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      if (row0) *reinterpret_cast<float2*>(pr0p + n * 8 + cl) = make_float2(O[n][0], O[n][1]);
      if (row1) *reinterpret_cast<float2*>(pr1p + n * 8 + cl) = make_float2(O[n][2], O[n][3]);
    }
    if ((lane & 3) == 0) {
      if (row0) { pr0p[D] = m0; pr0p[D + 1] = l0; }
      if (row1) { pr1p[D] = m1; pr1p[D + 1] = l1; }
    }
    return;
  }
  const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int col = head * D + n * 8 + cl;
    if (row0) {
      float x = O[n][0] * i0, y = O[n][1] * i0;
      if (a.gate) {
        const float* gp = a.gate + (size_t)(q0 + rl) * a.gate_ld + col;
        x *= 1.f / (1.f + expf(-gp[0])); y *= 1.f / (1.f + expf(-gp[1]));
      }
      *reinterpret_cast<uint32_t*>(a.out + (size_t)(q0 + rl) * H * D + col) = tm_pack(x, y);
    }
    if (row1) {
      float x = O[n][2] * i1, y = O[n][3] * i1;
      if (a.gate) {
        const float* gp = a.gate + (size_t)(q0 + rl + 8) * a.gate_ld + col;
        x *= 1.f / (1.f + expf(-gp[0])); y *= 1.f / (1.f + expf(-gp[1]));
      }
      *reinterpret_cast<uint32_t*>(a.out + (size_t)(q0 + rl + 8) * H * D + col) = tm_pack(x, y);
    }
  }
}

// out[t, h, :] = sum_z parts[t, h, z, :D] * exp(m_z - m) / sum_z l_z * exp(m_z - m), m = max_z m_z, times sigmoid(gate):
// a warp per (token, head), the parts added in ascending z.
template <int D>
__global__ void __launch_bounds__(128)
attention_talk_merge_kernel(TalkMmaArgs a) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)a.n_tokens * a.H) return;
  const int tok = (int)(item / a.H), h = (int)(item % a.H);
  // a padding row (no request behind it) has no parts: its output is zero
  int lo = 0, hi = a.n_req;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.cu_q[mid] <= tok) lo = mid; else hi = mid; }
  const bool live = tok < a.cu_q[a.n_req] && a.seq_lens[lo] > 0;
  const float* p = a.parts + (size_t)item * a.splits * (D + 2);
  float m = -INFINITY;
  if (live) for (int z = 0; z < a.splits; ++z) m = fmaxf(m, p[(size_t)z * (D + 2) + D]);
  constexpr int PER = (D + 31) / 32;
  float acc[PER], l = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) acc[j] = 0.f;
  if (live)
    for (int z = 0; z < a.splits; ++z) {
      const float* pz = p + (size_t)z * (D + 2);
      const float mz = pz[D];
      if (mz == -INFINITY) continue;               // a split that saw no key
      const float w = expf(mz - m);
      l += pz[D + 1] * w;
#pragma unroll
      for (int j = 0; j < PER; ++j) { const int c = lane + 32 * j; if (c < D) acc[j] = fmaf(pz[c], w, acc[j]); }
    }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = lane + 32 * j;
    if (c >= D) continue;
    float o = live ? acc[j] / l : 0.f;
    if (live && a.gate) o *= 1.f / (1.f + expf(-a.gate[(size_t)tok * a.gate_ld + h * D + c]));
    a.out[(size_t)tok * a.H * D + h * D + c] = __float2bfloat16_rn(o);
  }
}

static size_t tm_smem_bytes(int H, int G, int D, int NW, int gv_max) {
  return ((size_t)NW * TM_ROWS + (size_t)2 * gv_max * TM_KEYS) * (D + 8) * sizeof(bf16) +
         ((size_t)2 * NW * TM_ROWS * TM_KEYS + (size_t)H * NW) * sizeof(float);
}
static int tm_warps(int H) { return H <= 4 ? 4 : H <= 8 ? 8 : 16; }
static int tm_gv_max(int H, int G, int NW) {        // key/value heads that a group of NW query heads can touch
  const int rep = H / G;
  int most = 1;
  for (int o0 = 0; o0 < H; o0 += NW) {
    const int last = (o0 + NW < H ? o0 + NW : H) - 1;
    most = max(most, last / rep - o0 / rep + 1);
  }
  return most;
}

// Whether the tensor-core kernel takes these sizes (else the caller runs the plain one): bfloat16, head size 16, 32, 64
// or 128, and a tile's shared memory within an SM's.
IFB_EXPORT int ifb_attention_talk_mma_fits(int H, int G, int D) {
  if (H < 1 || G < 1 || H % G || (D != 16 && D != 32 && D != 64 && D != 128)) return 0;
  const int NW = tm_warps(H);
  if ((H + NW - 1) / NW > 8) return 0;                      // the groups of a tile are one cluster
  return tm_smem_bytes(H, G, D, NW, tm_gv_max(H, G, NW)) <= 220 * 1024 ? 1 : 0;
}

template <int D, int NW>
static int tm_launch(const TalkMmaArgs& a, cudaStream_t s) {
  const int gv_max = tm_gv_max(a.H, a.G, NW);
  const size_t smem = tm_smem_bytes(a.H, a.G, D, NW, gv_max);
  const int groups = (a.H + NW - 1) / NW;
  dim3 grid((a.n_tokens + TM_ROWS - 1) / TM_ROWS + a.n_req, groups, a.splits);
  int st;
  if (groups == 1) {
    IFB_ALLOW_SMEM((attention_talk_mma_kernel<D, NW, false>), smem);
    st = ifb_launch(attention_talk_mma_kernel<D, NW, false>, grid, dim3(NW * 32), smem, s, a, gv_max);
  } else {                                                  // the groups of a query tile: one cluster along y
    IFB_ALLOW_SMEM((attention_talk_mma_kernel<D, NW, true>), smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = groups;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ifb_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_talk_mma_kernel<D, NW, true>, a, gv_max);
    if (e != cudaSuccess) { cudaGetLastError(); return -(int)e; }
    st = IFB_OK;
  }
  if (st != IFB_OK || a.splits == 1) return st;
  const long long items = (long long)a.n_tokens * a.H;
  return ifb_launch(attention_talk_merge_kernel<D>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, a);
}

template <int D>
static int tm_by_heads(const TalkMmaArgs& a, cudaStream_t s) {
  switch (tm_warps(a.H)) {
    case 4: return tm_launch<D, 4>(a, s);
    case 8: return tm_launch<D, 8>(a, s);
    default: return tm_launch<D, 16>(a, s);
  }
}

// splits > 1 needs parts: n_tokens * H * splits * (d + 2) floats.
IFB_EXPORT int ifb_attention_talk_mma(const void* q, const void* pages, const int* block_tables, int bt_stride, const int* cu_q,
                                      const int* seq_lens, const void* talk, int talk_dtype, const float* gate, int gate_ld,
                                      void* out, int n_tokens, int n_req, int H, int G, int d, int page_size, int chunk,
                                      float scale, float slope_exp, int splits, float* parts, cudaStream_t stream) {
  if (n_tokens <= 0 || n_req <= 0) return IFB_OK;
  if (!ifb_attention_talk_mma_fits(H, G, d)) return IFB_ERR_SIZE;
  if (page_size < 1 || chunk < 0 || splits < 1 || splits > 64 || (splits > 1 && !parts)) return IFB_ERR_ARG;
  if (((uintptr_t)q & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3)) return IFB_ERR_ALIGN;
  if (gate && ((uintptr_t)gate & 3)) return IFB_ERR_ALIGN;
  if (talk && talk_dtype != IFB_F32 && talk_dtype != IFB_BF16) return IFB_ERR_DTYPE;
  TalkMmaArgs a{(const bf16*)q, (const bf16*)pages, block_tables, bt_stride, cu_q, seq_lens, talk, talk_dtype, gate, gate_ld,
                (bf16*)out, n_tokens, n_req, H, G, page_size, chunk, scale, slope_exp, splits, parts};
  switch (d) {
    case 16: return tm_by_heads<16>(a, stream);
    case 32: return tm_by_heads<32>(a, stream);
    case 64: return tm_by_heads<64>(a, stream);
    default: return tm_by_heads<128>(a, stream);
  }
}
