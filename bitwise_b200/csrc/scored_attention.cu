// Grouped-query softmax attention over paged keys and values with optional steps around the
// scores, and the kernels that prepare its operands.
//
//   qkv_prepare        per row and head: a short causal convolution over time on every channel of
//                      the projected q, k, v (inputs before the step's first row come from the
//                      request's state slot), a root-mean-square norm per head of q and k, the
//                      rotation of the leading entries of q and k (pair i = entries 2i, 2i + 1), q
//                      into the step's buffer, k and v into their pages
//   conv_state_update  the convolution's inputs of a request's last taps - 1 positions
//   scored_attention   s = (q . k) * scale; s <- cap * tanh(s / cap); s <- s - slope_h * (i - j);
//                      window; softmax with an optional extra one in the denominator; the values
//                      may be the keys themselves (no value pages)
//
// Everything after the projection is float32 in both precisions; only what is loaded and stored
// changes type. Keys are walked in tiles of 32 at fixed absolute positions, so what a query gets
// depends on its own keys only: not on the other rows of the step, nor on where a portion began.
#include "bw_act.cuh"
#include "bw_mma.cuh"

#include <math.h>

namespace {

// ---------------------------------------------------------------------------------------
// qkv_prepare. One block per row, a warp per head of q, k or v at a time; lane l holds the
// entries l, l + 32, ... of the head (up to kMaxE * 32).
constexpr int kMaxE = 8;
constexpr int kPrepWarps = 4;

struct PrepArgs {
  const float* u;            // [n, cols] projected rows: q heads, then k heads, then v heads
  int cols;
  const float* conv_w;       // [cols, taps] or null
  int taps;
  const float* conv_state;   // [slots, taps - 1, cols] or null
  const float* q_norm;       // [dim] or null
  const float* k_norm;
  float eps;
  const float* cos_t;        // [positions, pairs] or null
  const float* sin_t;
  int pairs;
  const int* pos;
  const int* row_seq;
  const int* seq_row0;
  const int* seq_pos0;
  const int* seq_slot;
  const int* block_table;
  int max_blocks;
  act_t* kcache;             // [pages, kv_heads, page, dim]
  act_t* vcache;             // [pages, kv_heads, page, vdim] or null
  act_t* q_out;              // [n, heads * dim]
  int heads, kv_heads /* 0: nothing is stored */, v_heads, dim, vdim, page;
};

__global__ void __launch_bounds__(kPrepWarps * 32) qkv_prepare_kernel(const PrepArgs a) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = a.pos[r];
  const int seq = a.row_seq[r];
  const int row0 = a.seq_row0[seq];
  const int slot = a.conv_state ? a.seq_slot[seq] : 0;
  const int total = a.heads + a.kv_heads + a.v_heads;
  for (int hs = warp; hs < total; hs += kPrepWarps) {
    int size, col0;
    const float* norm_w;
    bool turns;
    if (hs < a.heads) {
      size = a.dim, col0 = hs * a.dim, norm_w = a.q_norm, turns = true;
    } else if (hs < a.heads + a.kv_heads) {
      size = a.dim, col0 = hs * a.dim, norm_w = a.k_norm, turns = true;
    } else {
      size = a.vdim, col0 = (a.heads + a.kv_heads) * a.dim + (hs - a.heads - a.kv_heads) * a.vdim, norm_w = nullptr;
      turns = false;
    }
    float val[kMaxE];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxE; ++j) {
      const int e = lane + 32 * j;
      float v = 0.0f;
      if (e < size) {
        const int c = col0 + e;
        if (a.conv_w) {
          // y_t = sum_j w[c][j] * u_(t - taps + 1 + j), taps ascending; inputs before position 0 are zero
          for (int t = 0; t < a.taps; ++t) {
            const int back = a.taps - 1 - t;
            if (p - back < 0) continue;
            const int rr = r - back;
            const float src = rr >= row0
                                  ? a.u[static_cast<size_t>(rr) * a.cols + c]
                                  : a.conv_state[(static_cast<size_t>(slot) * (a.taps - 1) + (a.taps - 1 - (row0 - rr))) * a.cols + c];
            v = __fmaf_rn(a.conv_w[static_cast<size_t>(c) * a.taps + t], src, v);
          }
        } else {
          v = a.u[static_cast<size_t>(r) * a.cols + c];
        }
        ss = __fmaf_rn(v, v, ss);
      }
      val[j] = v;
    }
    if (norm_w) {
      const float inv = bw::rms_scale(bw::warp_sum(ss), size, a.eps);
#pragma unroll
      for (int j = 0; j < kMaxE; ++j) {
        const int e = lane + 32 * j;
        if (e < size) val[j] = bw::rms_apply(val[j], inv, norm_w[e]);
      }
    }
    if (turns && a.pairs > 0) {
#pragma unroll
      for (int j = 0; j < kMaxE; ++j) {
        const int e = lane + 32 * j;
        const float other = __shfl_xor_sync(0xffffffffu, val[j], 1);  // the partner of entry e is entry e ^ 1
        if (e < 2 * a.pairs && e < size) {
          const float c = a.cos_t[static_cast<size_t>(p) * a.pairs + (e >> 1)];
          const float s = a.sin_t[static_cast<size_t>(p) * a.pairs + (e >> 1)];
          val[j] = (e & 1) ? __fadd_rn(__fmul_rn(val[j], c), __fmul_rn(other, s))
                           : __fsub_rn(__fmul_rn(val[j], c), __fmul_rn(other, s));
        }
      }
    }
    act_t* dst;
    if (hs < a.heads) {
      dst = a.q_out + static_cast<size_t>(r) * a.heads * a.dim + hs * a.dim;
    } else {
      const int blk = a.block_table[static_cast<size_t>(seq) * a.max_blocks + p / a.page];
      if (hs < a.heads + a.kv_heads)
        dst = a.kcache + ((static_cast<size_t>(blk) * a.kv_heads + (hs - a.heads)) * a.page + p % a.page) * a.dim;
      else
        dst = a.vcache + ((static_cast<size_t>(blk) * a.v_heads + (hs - a.heads - a.kv_heads)) * a.page + p % a.page) * a.vdim;
    }
#pragma unroll
    for (int j = 0; j < kMaxE; ++j) {
      const int e = lane + 32 * j;
      if (e < size) dst[e] = bw::from_f<act_t>(val[j]);
    }
  }
}

// state[slot][i] = the projected row of position end - (taps - 1) + i (i < taps - 1), `end` the
// request's length after this step: from the step's rows, from the old state, or zero before
// position 0. One thread per (sequence, channel) reads all it needs before it writes.
constexpr int kMaxTaps = 16;

__global__ void __launch_bounds__(128)
conv_state_update_kernel(const float* __restrict__ u, int cols, float* state, int taps, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                         const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot) {
  bw::pdl_enter();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int seq = tile_seq[t], row0 = tile_row0[t], cnt = tile_rows[t];
  const int pos0 = seq_pos0[seq];
  float* st = state + static_cast<size_t>(seq_slot[seq]) * (taps - 1) * cols + c;
  float keep[kMaxTaps];
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
    if (i >= taps - 1) break;
    const int p = pos0 + cnt - (taps - 1) + i;
    float v = 0.0f;
    if (p >= pos0)
      v = u[static_cast<size_t>(row0 + p - pos0) * cols + c];
    else if (p >= 0)
      v = st[static_cast<size_t>(p - pos0 + taps - 1) * cols];
    keep[i] = v;
  }
#pragma unroll
  for (int i = 0; i < kMaxTaps; ++i) {
    if (i >= taps - 1) break;
    st[static_cast<size_t>(i) * cols] = keep[i];
  }
}

// ---------------------------------------------------------------------------------------
// Attention on the CUDA cores. A block takes one query tile (rows of one sequence at consecutive
// positions), one key/value head and up to `hb` of the query heads that read it; a warp works on
// one query (a row and a head) at a time, lane l on key l of the tile of 32: its score, the tile's
// maximum and sum over the warp, and the running (maximum, sum, weighted sum of values).
constexpr int kWarps = 8;
constexpr int kKeys = 32;
constexpr int kThreads = kWarps * 32;
constexpr int kQW = 4;  // queries per warp

struct ScoreArgs {
  float scale, softcap;
  int sink;
  const float* slopes;  // [heads] or null
  int window;
};

__device__ __forceinline__ float modify_score(float s, const ScoreArgs& sa, float slope, int pq, int kp) {
  s = __fmul_rn(s, sa.scale);
  if (sa.softcap > 0.0f) s = __fmul_rn(sa.softcap, tanhf(__fdiv_rn(s, sa.softcap)));
  if (sa.slopes) s = __fsub_rn(s, __fmul_rn(slope, static_cast<float>(pq - kp)));
  return s;
}

template <int ACC>
__global__ void __launch_bounds__(kThreads)
scored_attention_kernel(const act_t* __restrict__ q, int q_stride, const act_t* __restrict__ kcache,
                        const act_t* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                        const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                        const int* __restrict__ seq_row0, act_t* out, int o_stride, int heads, int kv_heads, int hb,
                        int dim, int vdim, int page, const ScoreArgs sa) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int ks = dim + 1;
  float* keys = sm;                                         // [32][dim + 1]
  float* vals = vcache ? keys + kKeys * ks : keys;          // [32][vdim], or the keys themselves
  const int vs = vcache ? vdim : ks;
  float* qs = keys + kKeys * ks + (vcache ? kKeys * vdim : 0);
  const int t = blockIdx.x, g = blockIdx.y;
  const int rep = heads / kv_heads;
  const int h0 = g * rep + blockIdx.z * hb;
  const int nh = min(hb, rep - blockIdx.z * hb);
  const int seq = tile_seq[t], row0 = tile_row0[t], rows = tile_rows[t];
  const int nq = rows * nh;
  const int p0 = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int qi = warp; qi < nq; qi += kWarps) {
    const act_t* src = q + static_cast<size_t>(row0 + qi / nh) * q_stride + (h0 + qi % nh) * dim;
    for (int d = lane; d < dim; d += 32) qs[qi * dim + d] = bw::to_f(src[d]);
  }
  float m[kQW], l[kQW], acc[kQW][ACC];
#pragma unroll
  for (int j = 0; j < kQW; ++j) {
    m[j] = -INFINITY, l[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[j][i] = 0.0f;
  }
  const int last = p0 + rows - 1;
  const int first = sa.window > 0 ? max(0, p0 - sa.window + 1) : 0;  // pages before it may be gone
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  for (int k0 = first / kKeys * kKeys; k0 <= last; k0 += kKeys) {
    __syncthreads();
    for (int kk = warp; kk < kKeys; kk += kWarps) {
      const int kp = k0 + kk;
      const bool have = kp <= last && kp >= first;
      size_t at = 0;
      if (have) at = (static_cast<size_t>(bt[kp / page]) * kv_heads + g) * page + kp % page;
      for (int d = lane; d < dim; d += 32) keys[kk * ks + d] = have ? bw::to_f(kcache[at * dim + d]) : 0.0f;
      if (vcache)
        for (int d = lane; d < vdim; d += 32) vals[kk * vs + d] = have ? bw::to_f(vcache[at * vdim + d]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kQW; ++j) {
      const int qi = warp + kWarps * j;
      if (qi >= nq) continue;
      const int pq = p0 + qi / nh;
      const int lo = sa.window > 0 ? max(0, pq - sa.window + 1) : 0;
      if (k0 > pq || k0 + kKeys <= lo) continue;  // no key of the tile is seen: the state stays
      const int kp = k0 + lane;
      const float* qv = qs + qi * dim;
      const float* kv = keys + lane * ks;
      float s = 0.0f;
      for (int d = 0; d < dim; ++d) s = __fmaf_rn(qv[d], kv[d], s);
      s = modify_score(s, sa, sa.slopes ? sa.slopes[h0 + qi % nh] : 0.0f, pq, kp);
      const bool seen = kp <= pq && kp >= lo;
      if (!seen) s = -INFINITY;
      const float mt = bw::warp_max(s);
      const float mn = fmaxf(m[j], mt);
      const float alpha = m[j] == -INFINITY ? 0.0f : expf(__fsub_rn(m[j], mn));
      const float pw = seen ? expf(__fsub_rn(s, mn)) : 0.0f;
      l[j] = __fmaf_rn(l[j], alpha, bw::warp_sum(pw));
#pragma unroll
      for (int i = 0; i < ACC; ++i) acc[j][i] = __fmul_rn(acc[j][i], alpha);
      for (int kk = 0; kk < kKeys; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, pw, kk);
        if (pk == 0.0f) continue;
        const float* vrow = vals + kk * vs;
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
          const int d = i * 32 + lane;
          if (d < vdim) acc[j][i] = __fmaf_rn(pk, vrow[d], acc[j][i]);
        }
      }
      m[j] = mn;
    }
  }
#pragma unroll
  for (int j = 0; j < kQW; ++j) {
    const int qi = warp + kWarps * j;
    if (qi >= nq) continue;
    float den = l[j];
    if (sa.sink) den = __fadd_rn(den, expf(-m[j]));  // the extra key of score 0
    const float inv = __fdiv_rn(1.0f, den);
    act_t* dst = out + static_cast<size_t>(row0 + qi / nh) * o_stride + (h0 + qi % nh) * vdim;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
      const int d = i * 32 + lane;
      if (d < vdim) dst[d] = bw::from_f<act_t>(__fmul_rn(acc[j][i], inv));
    }
  }
}

template <int ACC>
int launch_scored(dim3 grid, size_t smem, cudaStream_t stream, const act_t* q, int q_stride, const act_t* kcache,
                  const act_t* vcache, const int* block_table, int max_blocks, const int* tile_seq, const int* tile_row0,
                  const int* tile_rows, const int* seq_pos0, const int* seq_row0, act_t* out, int o_stride, int heads,
                  int kv_heads, int hb, int dim, int vdim, int page, const ScoreArgs& sa) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(scored_attention_kernel<ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("scored_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    allowed = smem;
  }
  bw::launch_pdl(scored_attention_kernel<ACC>, grid, dim3(kThreads), smem, stream, q, q_stride, kcache, vcache, block_table,
                 max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out, o_stride, heads, kv_heads, hb, dim,
                 vdim, page, sa);
  return bw::launch_status();
}

}  // namespace

// Rows of one sequence per query tile for `group` query heads on a key/value head.
BW_API int BW_FN(scored_attention_tile_rows)(int group) {
  const int hb = group < kWarps * kQW ? group : kWarps * kQW;
  return (kWarps * kQW) / (hb > 0 ? hb : 1);
}

BW_API int BW_FN(qkv_prepare)(const float* u, int cols, const float* conv_w, int taps, const float* conv_state,
                              const float* q_norm, const float* k_norm, float eps, const float* cos_t, const float* sin_t,
                              int pairs, const int* pos, const int* row_seq, const int* seq_row0, const int* seq_pos0,
                              const int* seq_slot, const int* block_table, int max_blocks, void* kcache, void* vcache,
                              void* q_out, int n, int heads, int kv_heads, int dim, int vdim, int page,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim > kMaxE * 32 || vdim > kMaxE * 32) {
    bw::set_error("qkv_prepare: head sizes %d / %d (up to %d)", dim, vdim, kMaxE * 32);
    return -1;
  }
  if (conv_w && taps > 1 && !conv_state) {
    bw::set_error("qkv_prepare: a convolution of %d taps needs the requests' state", taps);
    return -1;
  }
  PrepArgs a;
  a.u = u, a.cols = cols, a.conv_w = conv_w, a.taps = taps, a.conv_state = taps > 1 ? conv_state : nullptr;
  a.q_norm = q_norm, a.k_norm = k_norm, a.eps = eps, a.cos_t = cos_t, a.sin_t = sin_t, a.pairs = cos_t ? pairs : 0;
  a.pos = pos, a.row_seq = row_seq, a.seq_row0 = seq_row0, a.seq_pos0 = seq_pos0, a.seq_slot = seq_slot;
  a.block_table = block_table, a.max_blocks = max_blocks;
  a.kcache = static_cast<act_t*>(kcache), a.vcache = static_cast<act_t*>(vcache), a.q_out = static_cast<act_t*>(q_out);
  a.heads = heads, a.kv_heads = kv_heads, a.v_heads = vcache ? kv_heads : 0, a.dim = dim, a.vdim = vdim, a.page = page;
  bw::launch_pdl(qkv_prepare_kernel, dim3(n), dim3(kPrepWarps * 32), 0, stream, a);
  return bw::launch_status();
}

BW_API int BW_FN(conv_state_update)(const float* u, int cols, float* state, int taps, const int* tile_seq,
                                    const int* tile_row0, const int* tile_rows, int tiles, const int* seq_pos0,
                                    const int* seq_slot, cudaStream_t stream) {
  if (tiles <= 0 || taps <= 1) return 0;
  if (taps - 1 > kMaxTaps) {
    bw::set_error("conv_state_update: %d taps (up to %d)", taps, kMaxTaps + 1);
    return -1;
  }
  bw::launch_pdl(conv_state_update_kernel, dim3(tiles, (cols + 127) / 128), dim3(128), 0, stream, u, cols, state, taps,
                 tile_seq, tile_row0, tile_rows, seq_pos0, seq_slot);
  return bw::launch_status();
}

BW_API int BW_FN(scored_attention)(const void* q, int q_stride, const void* kcache, const void* vcache,
                                   const int* block_table, int max_blocks, const int* tile_seq, const int* tile_row0,
                                   const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_row0, void* out,
                                   int o_stride, int heads, int kv_heads, int dim, int vdim, int page, float scale,
                                   float softcap, int sink, const float* slopes, int window, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads) {
    bw::set_error("scored_attention: %d heads on %d key/value heads", heads, kv_heads);
    return -1;
  }
  const int acc = (vdim + 31) / 32;
  if (acc > 8) {
    bw::set_error("scored_attention: value size %d (up to 256)", vdim);
    return -1;
  }
  const int rep = heads / kv_heads;
  const int hb = rep < kWarps * kQW ? rep : kWarps * kQW;
  const size_t smem = (static_cast<size_t>(kKeys) * (dim + 1) + (vcache ? static_cast<size_t>(kKeys) * vdim : 0) +
                       static_cast<size_t>(kWarps * kQW) * dim) * sizeof(float);
  if (smem > 200 * 1024) {
    bw::set_error("scored_attention: head sizes %d / %d need %zu bytes of shared memory", dim, vdim, smem);
    return -1;
  }
  ScoreArgs sa;
  sa.scale = scale, sa.softcap = softcap, sa.sink = sink, sa.slopes = slopes, sa.window = window;
  const dim3 grid(tiles, kv_heads, (rep + hb - 1) / hb);
#define BW_SCORED(A)                                                                                                      \
  case A:                                                                                                                 \
    return launch_scored<A>(grid, smem, stream, static_cast<const act_t*>(q), q_stride, static_cast<const act_t*>(kcache), \
                            static_cast<const act_t*>(vcache), block_table, max_blocks, tile_seq, tile_row0, tile_rows,   \
                            seq_pos0, seq_row0, static_cast<act_t*>(out), o_stride, heads, kv_heads, hb, dim, vdim, page, \
                            sa);
  switch (acc) {
    BW_SCORED(1) BW_SCORED(2) BW_SCORED(3) BW_SCORED(4) BW_SCORED(5) BW_SCORED(6) BW_SCORED(7) BW_SCORED(8)
  }
#undef BW_SCORED
  return -1;
}
