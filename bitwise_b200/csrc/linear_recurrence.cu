// Gated linear attention: per head a state S of dim x vdim float32 numbers per request,
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t + b) ^ (1 / tau),
// followed by the root-mean-square norm of o_t over vdim (times a weight) and the gate silu(g_t).
//
// A block walks the rows of one sequence of the step for one head, token by token, from the
// state that the request's slot holds (zero at a request's first position). Thread (p, j) keeps
// rows p R .. p R + R - 1 of column j of S in registers; the tokens' q, k, a and v are staged in
// shared memory a chunk at a time, and the partial outputs of the row partitions are added in the
// order of p. The chunk is a staging unit only: every S_t and o_t is the same chain of operations
// wherever the step's rows begin and end, so a position's result does not depend on the cut.
// Everything here is float32 in both precisions; only the gated output changes type.
#include "bw_act.cuh"

#include <math.h>

namespace {

constexpr int kChunk = 8;  // tokens staged at a time

// log(sigmoid(x)) without overflow: min(x, 0) - log1p(exp(-|x|)).
__device__ __forceinline__ float log_sigmoid(float x) { return __fsub_rn(fminf(x, 0.0f), log1pf(expf(-fabsf(x)))); }

struct ScanArgs {
  const float* u;       // [n, stride]: q heads | k heads | v heads | gate
  int stride;
  const float* z;       // [n, heads * dim]
  const float* bias;    // [heads * dim]
  float inv_tau;
  float* state;         // [slots, heads, dim, vdim]
  const float* norm_w;  // [vdim]
  float eps;
  act_t* out;           // [n, heads * vdim]
  const int* tile_seq;
  const int* tile_row0;
  const int* tile_rows;
  const int* seq_pos0;
  const int* seq_slot;
  int heads, dim, vdim, parts;
  float q_scale;
};

template <int R, int T /* the most threads a block of this variant has: bounds its registers */>
__global__ void __launch_bounds__(T) gla_scan_kernel(const ScanArgs a) {
  bw::pdl_enter();
  extern __shared__ float sm[];
  const int dim = a.dim, vdim = a.vdim, P = a.parts;
  float* qs = sm;                      // [kChunk][dim]
  float* ks = qs + kChunk * dim;       // [kChunk][dim]
  float* as = ks + kChunk * dim;       // [kChunk][dim]
  float* vs = as + kChunk * dim;       // [kChunk][vdim]
  float* part = vs + kChunk * vdim;    // [kChunk][P][vdim]
  float* os = part + kChunk * P * vdim;  // [kChunk][vdim]
  const int t = blockIdx.x, h = blockIdx.y;
  const int seq = a.tile_seq[t], row0 = a.tile_row0[t], cnt = a.tile_rows[t];
  const int tid = threadIdx.x, threads = blockDim.x;
  const int j = tid % vdim, p = tid / vdim;
  const bool owner = p < P;
  const int hd = a.heads * dim, hv = a.heads * vdim;
  float* sp = a.state + ((static_cast<size_t>(a.seq_slot[seq]) * a.heads + h) * dim) * vdim;
  float S[R];
  const bool fresh = a.seq_pos0[seq] == 0;  // a slot is handed out as its last holder left it
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = p * R + i;
    S[i] = (!fresh && owner && row < dim) ? sp[static_cast<size_t>(row) * vdim + j] : 0.0f;
  }
  for (int c0 = 0; c0 < cnt; c0 += kChunk) {
    const int len = min(kChunk, cnt - c0);
    __syncthreads();
    for (int i = tid; i < len * dim; i += threads) {
      const int tt = i / dim, d = i - tt * dim;
      const size_t r = static_cast<size_t>(row0 + c0 + tt);
      qs[i] = __fmul_rn(a.u[r * a.stride + h * dim + d], a.q_scale);
      ks[i] = a.u[r * a.stride + hd + h * dim + d];
      const float zz = __fadd_rn(a.z[r * hd + h * dim + d], a.bias[h * dim + d]);
      as[i] = expf(__fmul_rn(log_sigmoid(zz), a.inv_tau));
    }
    for (int i = tid; i < len * vdim; i += threads) {
      const int tt = i / vdim, d = i - tt * vdim;
      vs[i] = a.u[static_cast<size_t>(row0 + c0 + tt) * a.stride + 2 * hd + h * vdim + d];
    }
    __syncthreads();
    if (owner) {
      for (int tt = 0; tt < len; ++tt) {
        const float v = vs[tt * vdim + j];
        const float* qt = qs + tt * dim + p * R;
        const float* kt = ks + tt * dim + p * R;
        const float* at = as + tt * dim + p * R;
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          if (p * R + i < dim) {
            S[i] = __fmaf_rn(at[i], S[i], __fmul_rn(kt[i], v));
            o = __fmaf_rn(qt[i], S[i], o);
          }
        }
        part[(tt * P + p) * vdim + j] = o;
      }
    }
    __syncthreads();
    for (int i = tid; i < len * vdim; i += threads) {
      const int tt = i / vdim, d = i - tt * vdim;
      float o = 0.0f;
      for (int pp = 0; pp < P; ++pp) o = __fadd_rn(o, part[(tt * P + pp) * vdim + d]);
      os[i] = o;
    }
    __syncthreads();
    // the norm over vdim and the gate: a warp per token
    const int warp = tid >> 5, lane = tid & 31, warps = (threads + 31) >> 5;
    for (int tt = warp; tt < len; tt += warps) {
      float ss = 0.0f;
      for (int d = lane; d < vdim; d += 32) ss = __fmaf_rn(os[tt * vdim + d], os[tt * vdim + d], ss);
      const float inv = bw::rms_scale(bw::warp_sum(ss), vdim, a.eps);
      const size_t r = static_cast<size_t>(row0 + c0 + tt);
      for (int d = lane; d < vdim; d += 32) {
        const float g = a.u[r * a.stride + 2 * hd + hv + h * vdim + d];
        const float gate = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
        a.out[r * hv + h * vdim + d] = bw::from_f<act_t>(__fmul_rn(bw::rms_apply(os[tt * vdim + d], inv, a.norm_w[d]), gate));
      }
    }
  }
  if (owner) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = p * R + i;
      if (row < dim) sp[static_cast<size_t>(row) * vdim + j] = S[i];
    }
  }
}

template <int R, int T>
int launch_scan_t(const ScanArgs& a, int tiles, int threads, size_t smem, cudaStream_t stream) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<R, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("gla_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    allowed = smem;
  }
  bw::launch_pdl(gla_scan_kernel<R, T>, dim3(tiles, a.heads), dim3(threads), smem, stream, a);
  return bw::launch_status();
}

template <int R>
int launch_scan(const ScanArgs& a, int tiles, int threads, size_t smem, cudaStream_t stream) {
  if (threads <= 256) return launch_scan_t<R, 256>(a, tiles, threads, smem, stream);
  if (threads <= 512) return launch_scan_t<R, 512>(a, tiles, threads, smem, stream);
  return launch_scan_t<R, 1024>(a, tiles, threads, smem, stream);
}

}  // namespace

BW_API int BW_FN(gla_scan)(const float* u, int stride, const float* z, const float* bias, float tau, float* state,
                           const float* norm_w, float eps, void* out, const int* tile_seq, const int* tile_row0,
                           const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_slot, int heads, int dim,
                           int vdim, float q_scale, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (vdim > 1024 || dim > 64 * (1024 / vdim)) {
    bw::set_error("gla_scan: a state of %d x %d per head does not fit a block's registers", dim, vdim);
    return -1;
  }
  // The fewest state rows per thread for which the block stays within 1,024 threads and its
  // threads within the registers of an SM (the rows and about 40 more each); where no choice
  // does, the fewest rows that fit the thread limit (the compiler then spills some of the rows).
  int rows = 0;
  for (int r = 8; r <= 64 && !rows; r *= 2) {
    const int th = (dim + r - 1) / r * vdim;
    if (th <= 1024 && (r + 40) * th <= 65536) rows = r;
  }
  for (int r = 8; r <= 64 && !rows; r *= 2)
    if ((dim + r - 1) / r * vdim <= 1024) rows = r;
  ScanArgs a;
  a.u = u, a.stride = stride, a.z = z, a.bias = bias, a.inv_tau = 1.0f / tau, a.state = state, a.norm_w = norm_w, a.eps = eps;
  a.out = static_cast<act_t*>(out), a.tile_seq = tile_seq, a.tile_row0 = tile_row0, a.tile_rows = tile_rows;
  a.seq_pos0 = seq_pos0, a.seq_slot = seq_slot, a.heads = heads, a.dim = dim, a.vdim = vdim, a.q_scale = q_scale;
  a.parts = (dim + rows - 1) / rows;
  int threads = a.parts * vdim;
  threads = (threads + 31) / 32 * 32;
  const size_t smem = static_cast<size_t>(kChunk) * (3 * dim + vdim + a.parts * vdim + vdim) * sizeof(float);
  if (smem > 200 * 1024) {
    bw::set_error("gla_scan: head sizes %d / %d need %zu bytes of shared memory", dim, vdim, smem);
    return -1;
  }
  switch (rows) {
    case 8: return launch_scan<8>(a, tiles, threads, smem, stream);
    case 16: return launch_scan<16>(a, tiles, threads, smem, stream);
    case 32: return launch_scan<32>(a, tiles, threads, smem, stream);
    case 64: return launch_scan<64>(a, tiles, threads, smem, stream);
  }
  bw::set_error("gla_scan: %d state rows per thread", rows);
  return -1;
}
