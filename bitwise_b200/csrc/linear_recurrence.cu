// Gated linear attention: per head a state S of dim x vdim float32 numbers per request,
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t + b) ^ (1 / tau),
// followed by the root-mean-square norm of o_t over vdim (times a weight) and the gate silu(g_t).
//
// The columns of S do not meet before the norm, so a block walks the rows of one sequence of the
// step for one head and 8 value columns, token by token, from the state that the request's slot
// holds (zero at a request's first position). Thread (p, j) keeps rows p R .. p R + R - 1 of
// column j in registers. The tokens' q, k, z and v are copied into shared memory a chunk ahead
// (cp.async, two buffers), the decays are formed there, and the partial outputs of the row
// partitions are added in the order of p. The chunk is a staging unit only: every S_t and o_t is
// the same chain of operations wherever the step's rows begin and end, so a position's result
// does not depend on the cut. A second kernel norms every head's o over vdim and applies the gate.
// Everything here is float32 in both precisions; only the gated output changes type.
#include "bw_act.cuh"

#include <math.h>

namespace {

constexpr int kCols = 8;      // value columns per block: a head's columns are spread over many blocks
constexpr int kMaxThreads = 256;

// log(sigmoid(x)) without overflow: min(x, 0) - log1p(exp(-|x|)). The serving precision takes the
// hardware's exponential and logarithm (relative error about 1e-7, far below a bfloat16 operand's).
__device__ __forceinline__ float decay_of(float x, float inv_tau) {
#if BW_ACT_BF16
  const float ls = __fsub_rn(fminf(x, 0.0f), __logf(__fadd_rn(1.0f, __expf(-fabsf(x)))));
  return __expf(__fmul_rn(ls, inv_tau));
#else
  const float ls = __fsub_rn(fminf(x, 0.0f), log1pf(expf(-fabsf(x))));
  return expf(__fmul_rn(ls, inv_tau));
#endif
}

__device__ __forceinline__ void copy4_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void copy16_async(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copies_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

struct ScanArgs {
  const float* u;       // [n, stride]: q heads | k heads | v heads | gate
  int stride;
  const float* z;       // [n, heads * dim]
  const float* bias;    // [heads * dim]
  float inv_tau;
  float* state;         // [slots, heads, dim, vdim]
  float* o;             // [n, heads * vdim]: the recurrence's outputs before their norm
  const int* tile_seq;
  const int* tile_row0;
  const int* tile_rows;
  const int* seq_pos0;
  const int* seq_slot;
  int heads, dim, vdim, parts, chunk;
  float q_scale;
};

// Thread (p, j): rows p R .. p R + R - 1 of column c0 + j of S. R is 2, 4, 8 or 16.
template <int R, bool VEC /* dim is a multiple of 4: a thread's q, k and decays are read as vectors */>
__global__ void __launch_bounds__(kMaxThreads) gla_scan_kernel(const ScanArgs a) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float sm[];
  const int dim = a.dim, vdim = a.vdim, P = a.parts, chunk = a.chunk;
  const int W = 3 * dim + kCols;                 // a staged token: q | k | z (then the decay) | 8 values
  float* stage = sm;                             // [2][chunk][W]
  float* part = sm + 2 * chunk * W;              // [chunk][P][kCols]
  const int t = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kCols;
  const int seq = a.tile_seq[t], row0 = a.tile_row0[t], cnt = a.tile_rows[t];
  const int tid = threadIdx.x, threads = blockDim.x;
  const int j = tid & (kCols - 1), p = tid / kCols;
  const bool col_ok = c0 + j < vdim;
  const int hd = a.heads * dim, hv = a.heads * vdim;
  float* sp = a.state + ((static_cast<size_t>(a.seq_slot[seq]) * a.heads + h) * dim) * vdim + c0 + j;
  float S[R];
  const bool fresh = a.seq_pos0[seq] == 0;  // a slot is handed out as its last holder left it
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = p * R + i;
    S[i] = (!fresh && col_ok && p < P && row < dim) ? sp[static_cast<size_t>(row) * vdim] : 0.0f;
  }
  // (16 bytes at a time where every row and head starts on 16 bytes)
  const bool wide = VEC && (vdim & 3) == 0 && (a.stride & 3) == 0 &&
                    ((reinterpret_cast<uintptr_t>(a.u) | reinterpret_cast<uintptr_t>(a.z)) & 15) == 0;
  auto request = [&](int first, float* buf) {
    const int len = min(chunk, cnt - first);
    const int step = wide ? 4 : 1;
    const int Ws = W / step;
    for (int i = tid; i < len * Ws; i += threads) {
      const int tt = i / Ws, e = (i - tt * Ws) * step;
      const size_t r = static_cast<size_t>(row0 + first + tt);
      const float* src;
      if (e < dim) src = a.u + r * a.stride + h * dim + e;
      else if (e < 2 * dim) src = a.u + r * a.stride + hd + h * dim + (e - dim);
      else if (e < 3 * dim) src = a.z + r * hd + h * dim + (e - 2 * dim);
      else if (c0 + e - 3 * dim < vdim) src = a.u + r * a.stride + 2 * hd + h * vdim + c0 + (e - 3 * dim);
      else continue;
      if (wide) copy16_async(buf + tt * W + e, src);
      else copy4_async(buf + tt * W + e, src);
    }
    copies_commit();
  };
  request(0, stage);
  for (int first = 0, b = 0; first < cnt; first += chunk, b ^= 1) {
    const int len = min(chunk, cnt - first);
    float* buf = stage + b * chunk * W;
    __syncthreads();  // the other buffer and `part` have been used
    if (first + chunk < cnt) {
      request(first + chunk, stage + (b ^ 1) * chunk * W);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    for (int i = tid; i < len * dim; i += threads) {
      const int tt = i / dim, d = i - tt * dim;
      float* tok = buf + tt * W;
      tok[d] = __fmul_rn(tok[d], a.q_scale);
      tok[2 * dim + d] = decay_of(__fadd_rn(tok[2 * dim + d], a.bias[h * dim + d]), a.inv_tau);
    }
    __syncthreads();
    if (p < P) {
#pragma unroll 2
      for (int tt = 0; tt < len; ++tt) {
        const float* tok = buf + tt * W;
        const float v = col_ok ? tok[3 * dim + j] : 0.0f;
        const float* qt = tok + p * R;
        const float* kt = tok + dim + p * R;
        const float* at = tok + 2 * dim + p * R;
        float qv[R], kv[R], av[R];
        if (VEC && R >= 4) {
#pragma unroll
          for (int i = 0; i < R; i += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qt + i), k4 = *reinterpret_cast<const float4*>(kt + i),
                         a4 = *reinterpret_cast<const float4*>(at + i);
            qv[i] = q4.x, qv[i + 1] = q4.y, qv[i + 2] = q4.z, qv[i + 3] = q4.w;
            kv[i] = k4.x, kv[i + 1] = k4.y, kv[i + 2] = k4.z, kv[i + 3] = k4.w;
            av[i] = a4.x, av[i + 1] = a4.y, av[i + 2] = a4.z, av[i + 3] = a4.w;
          }
        } else if (VEC && R == 2) {
          const float2 q2 = *reinterpret_cast<const float2*>(qt), k2 = *reinterpret_cast<const float2*>(kt),
                       a2 = *reinterpret_cast<const float2*>(at);
          qv[0] = q2.x, qv[1] = q2.y, kv[0] = k2.x, kv[1] = k2.y, av[0] = a2.x, av[1] = a2.y;
        } else {
#pragma unroll
          for (int i = 0; i < R; ++i) {
            const bool in = p * R + i < dim;
            qv[i] = in ? qt[i] : 0.0f, kv[i] = in ? kt[i] : 0.0f, av[i] = in ? at[i] : 0.0f;
          }
        }
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          if (VEC || p * R + i < dim) {  // (with VEC, R divides dim: every row of a partition exists)
            S[i] = __fmaf_rn(av[i], S[i], __fmul_rn(kv[i], v));
            o = __fmaf_rn(qv[i], S[i], o);
          }
        }
        part[(tt * P + p) * kCols + j] = o;
      }
    }
    __syncthreads();
    for (int i = tid; i < len * kCols; i += threads) {
      const int tt = i / kCols, c = i - tt * kCols;
      if (c0 + c >= vdim) continue;
      float o = 0.0f;
      for (int pp = 0; pp < P; ++pp) o = __fadd_rn(o, part[(tt * P + pp) * kCols + c]);
      a.o[static_cast<size_t>(row0 + first + tt) * hv + h * vdim + c0 + c] = o;
    }
  }
  if (p < P && col_ok) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = p * R + i;
      if (row < dim) sp[static_cast<size_t>(row) * vdim] = S[i];
    }
  }
}

// out[r, h] = o[r, h] / sqrt(mean(o[r, h]^2) + eps) * w * silu(gate[r, h]): a block per row, a warp per head.
__global__ void __launch_bounds__(128)
gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ u, int stride, int gate_col,
                  const float* __restrict__ w, float eps, act_t* out, int heads, int vdim) {
  bw::pdl_enter();
  const size_t r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hv = heads * vdim;
  for (int h = warp; h < heads; h += 4) {
    const float* oh = o + r * hv + h * vdim;
    float ss = 0.0f;
    for (int d = lane; d < vdim; d += 32) ss = __fmaf_rn(oh[d], oh[d], ss);
    const float inv = bw::rms_scale(bw::warp_sum(ss), vdim, eps);
    for (int d = lane; d < vdim; d += 32) {
      const float g = u[r * stride + gate_col + h * vdim + d];
      const float gate = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
      out[r * hv + h * vdim + d] = bw::from_f<act_t>(__fmul_rn(bw::rms_apply(oh[d], inv, w[d]), gate));
    }
  }
}

template <int R, bool VEC>
int launch_scan_v(const ScanArgs& a, int tiles, int threads, size_t smem, cudaStream_t stream) {
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<R, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) {
      bw::set_error("gla_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    allowed = smem;
  }
  bw::launch_pdl(gla_scan_kernel<R, VEC>, dim3(tiles, a.heads, (a.vdim + kCols - 1) / kCols), dim3(threads), smem, stream, a);
  return bw::launch_status();
}

template <int R>
int launch_scan(const ScanArgs& a, int tiles, int threads, size_t smem, cudaStream_t stream) {
  // (the order of a column's operations is the same either way: the same bits)
  return a.dim % 4 == 0 && a.dim % R == 0 ? launch_scan_v<R, true>(a, tiles, threads, smem, stream)
                                          : launch_scan_v<R, false>(a, tiles, threads, smem, stream);
}

}  // namespace

// `o32`: scratch [n, heads * vdim] float32 for the outputs before their norm.
BW_API int BW_FN(gla_scan)(const float* u, int stride, const float* z, const float* bias, float tau, float* state,
                           const float* norm_w, float eps, float* o32, void* out, const int* tile_seq, const int* tile_row0,
                           const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_slot, int n, int heads,
                           int dim, int vdim, float q_scale, cudaStream_t stream) {
  if (tiles <= 0 || n <= 0) return 0;
  // state rows per thread: the fewest of 2, 4, 8, 16 with which a block stays within 256 threads
  int rows = 2;
  while (rows < 16 && (dim + rows - 1) / rows * kCols > kMaxThreads) rows *= 2;
  ScanArgs a;
  a.u = u, a.stride = stride, a.z = z, a.bias = bias, a.inv_tau = 1.0f / tau, a.state = state, a.o = o32;
  a.tile_seq = tile_seq, a.tile_row0 = tile_row0, a.tile_rows = tile_rows;
  a.seq_pos0 = seq_pos0, a.seq_slot = seq_slot, a.heads = heads, a.dim = dim, a.vdim = vdim, a.q_scale = q_scale;
  a.parts = (dim + rows - 1) / rows;
  if (a.parts * kCols > kMaxThreads) {
    bw::set_error("gla_scan: key size %d (up to %d)", dim, 16 * kMaxThreads / kCols);
    return -1;
  }
  const int threads = (a.parts * kCols + 31) / 32 * 32;
  // Tokens staged at a time: no more than the longest sequence of the step can have (a step of
  // single rows stages one, so that many of its small blocks share an SM), and as many of 32 as
  // let two blocks share an SM's shared memory.
  int longest = n - tiles + 1;
  a.chunk = 1;
  while (a.chunk < 32 && a.chunk < longest) a.chunk *= 2;
  auto bytes = [&](int chunk) {
    return (static_cast<size_t>(2 * chunk) * (3 * dim + kCols) + static_cast<size_t>(chunk) * a.parts * kCols) * sizeof(float);
  };
  while (a.chunk > 4 && bytes(a.chunk) > 100 * 1024) a.chunk /= 2;
  const size_t smem = bytes(a.chunk);
  int rc = -1;
  switch (rows) {
    case 2: rc = launch_scan<2>(a, tiles, threads, smem, stream); break;
    case 4: rc = launch_scan<4>(a, tiles, threads, smem, stream); break;
    case 8: rc = launch_scan<8>(a, tiles, threads, smem, stream); break;
    case 16: rc = launch_scan<16>(a, tiles, threads, smem, stream); break;
  }
  if (rc != 0) return rc;
  bw::launch_pdl(gla_finish_kernel, dim3(n), dim3(128), 0, stream, static_cast<const float*>(o32), u, stride,
                 2 * heads * dim + heads * vdim, norm_w, eps, static_cast<act_t*>(out), heads, vdim);
  return bw::launch_status();
}
