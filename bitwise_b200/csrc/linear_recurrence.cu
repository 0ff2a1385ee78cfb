// Gated linear attention: per head a state S of dim x vdim float32 numbers per request,
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t + b) ^ (1 / tau),
// followed by the root-mean-square norm of o_t over vdim (times a weight) and the gate silu(g_t).
//
// The columns of S do not meet before the norm, so a block walks the rows of one sequence of the
// step for one head and 32 value columns, token by token, from the state that the request's slot
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

constexpr int kChunk = 32;   // tokens staged at a time
constexpr int kCols = 32;    // value columns per block
constexpr int kMaxParts = 8; // row partitions per block

// log(sigmoid(x)) without overflow: min(x, 0) - log1p(exp(-|x|)).
__device__ __forceinline__ float log_sigmoid(float x) { return __fsub_rn(fminf(x, 0.0f), log1pf(expf(-fabsf(x)))); }

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
  int heads, dim, vdim, parts;
  float q_scale;
};

template <int R, bool VEC /* dim is a multiple of 4: a partition's q, k and decays are read 16 bytes at a time */>
__global__ void __launch_bounds__(kMaxParts * kCols) gla_scan_kernel(const ScanArgs a) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float sm[];
  const int dim = a.dim, vdim = a.vdim, P = a.parts;
  const int W = 3 * dim + kCols;                 // a staged token: q | k | z (then the decay) | 32 values
  float* stage = sm;                             // [2][kChunk][W]
  float* part = sm + 2 * kChunk * W;             // [kChunk][P][kCols]
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
    S[i] = (!fresh && col_ok && row < dim) ? sp[static_cast<size_t>(row) * vdim] : 0.0f;
  }
  // (16 bytes at a time where every row and head starts on 16 bytes)
  const bool wide = VEC && (vdim & 3) == 0 && (a.stride & 3) == 0 &&
                    ((reinterpret_cast<uintptr_t>(a.u) | reinterpret_cast<uintptr_t>(a.z)) & 15) == 0;
  auto request = [&](int first, float* buf) {
    const int len = min(kChunk, cnt - first);
    if (wide) {
      const int W4 = W >> 2;
      for (int i = tid; i < len * W4; i += threads) {
        const int tt = i / W4, e = (i - tt * W4) << 2;
        const size_t r = static_cast<size_t>(row0 + first + tt);
        const float* src;
        if (e < dim) src = a.u + r * a.stride + h * dim + e;
        else if (e < 2 * dim) src = a.u + r * a.stride + hd + h * dim + (e - dim);
        else if (e < 3 * dim) src = a.z + r * hd + h * dim + (e - 2 * dim);
        else if (c0 + e - 3 * dim < vdim) src = a.u + r * a.stride + 2 * hd + h * vdim + c0 + (e - 3 * dim);
        else continue;
        copy16_async(buf + tt * W + e, src);
      }
      copies_commit();
      return;
    }
    for (int i = tid; i < len * W; i += threads) {
      const int tt = i / W, e = i - tt * W;
      const size_t r = static_cast<size_t>(row0 + first + tt);
      const float* src;
      if (e < dim) src = a.u + r * a.stride + h * dim + e;
      else if (e < 2 * dim) src = a.u + r * a.stride + hd + h * dim + (e - dim);
      else if (e < 3 * dim) src = a.z + r * hd + h * dim + (e - 2 * dim);
      else if (c0 + e - 3 * dim < vdim) src = a.u + r * a.stride + 2 * hd + h * vdim + c0 + (e - 3 * dim);
      else continue;
      copy4_async(buf + i, src);
    }
    copies_commit();
  };
  request(0, stage);
  for (int first = 0, b = 0; first < cnt; first += kChunk, b ^= 1) {
    const int len = min(kChunk, cnt - first);
    float* buf = stage + b * kChunk * W;
    __syncthreads();  // the other buffer and `part` have been used
    if (first + kChunk < cnt) {
      request(first + kChunk, stage + (b ^ 1) * kChunk * W);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    for (int i = tid; i < len * dim; i += threads) {
      const int tt = i / dim, d = i - tt * dim;
      float* tok = buf + tt * W;
      tok[d] = __fmul_rn(tok[d], a.q_scale);
      tok[2 * dim + d] = expf(__fmul_rn(log_sigmoid(__fadd_rn(tok[2 * dim + d], a.bias[h * dim + d])), a.inv_tau));
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
        float o = 0.0f;
        if (VEC) {
#pragma unroll
          for (int i = 0; i < R; i += 4) {
            if (p * R + i < dim) {
              const float4 q4 = *reinterpret_cast<const float4*>(qt + i), k4 = *reinterpret_cast<const float4*>(kt + i),
                           a4 = *reinterpret_cast<const float4*>(at + i);
              S[i] = __fmaf_rn(a4.x, S[i], __fmul_rn(k4.x, v)), o = __fmaf_rn(q4.x, S[i], o);
              S[i + 1] = __fmaf_rn(a4.y, S[i + 1], __fmul_rn(k4.y, v)), o = __fmaf_rn(q4.y, S[i + 1], o);
              S[i + 2] = __fmaf_rn(a4.z, S[i + 2], __fmul_rn(k4.z, v)), o = __fmaf_rn(q4.z, S[i + 2], o);
              S[i + 3] = __fmaf_rn(a4.w, S[i + 3], __fmul_rn(k4.w, v)), o = __fmaf_rn(q4.w, S[i + 3], o);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < R; ++i) {
            if (p * R + i < dim) {
              S[i] = __fmaf_rn(at[i], S[i], __fmul_rn(kt[i], v));
              o = __fmaf_rn(qt[i], S[i], o);
            }
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
  return a.dim % 4 == 0 ? launch_scan_v<R, true>(a, tiles, threads, smem, stream)
                        : launch_scan_v<R, false>(a, tiles, threads, smem, stream);
}

}  // namespace

// `o32`: scratch [n, heads * vdim] float32 for the outputs before their norm.
BW_API int BW_FN(gla_scan)(const float* u, int stride, const float* z, const float* bias, float tau, float* state,
                           const float* norm_w, float eps, float* o32, void* out, const int* tile_seq, const int* tile_row0,
                           const int* tile_rows, int tiles, const int* seq_pos0, const int* seq_slot, int n, int heads,
                           int dim, int vdim, float q_scale, cudaStream_t stream) {
  if (tiles <= 0 || n <= 0) return 0;
  // state rows per thread: the fewest of 8, 16, 32, 64 with which eight partitions cover the head
  int rows = 8;
  while (rows < 64 && (dim + rows - 1) / rows > kMaxParts) rows *= 2;
  ScanArgs a;
  a.u = u, a.stride = stride, a.z = z, a.bias = bias, a.inv_tau = 1.0f / tau, a.state = state, a.o = o32;
  a.tile_seq = tile_seq, a.tile_row0 = tile_row0, a.tile_rows = tile_rows;
  a.seq_pos0 = seq_pos0, a.seq_slot = seq_slot, a.heads = heads, a.dim = dim, a.vdim = vdim, a.q_scale = q_scale;
  a.parts = (dim + rows - 1) / rows;
  if (a.parts > kMaxParts) {
    bw::set_error("gla_scan: key size %d (up to %d)", dim, 64 * kMaxParts);
    return -1;
  }
  const int threads = a.parts * kCols;
  const size_t smem = (static_cast<size_t>(2 * kChunk) * (3 * dim + kCols) + static_cast<size_t>(kChunk) * a.parts * kCols) * sizeof(float);
  if (smem > 200 * 1024) {
    bw::set_error("gla_scan: key size %d needs %zu bytes of shared memory", dim, smem);
    return -1;
  }
  int rc = -1;
  switch (rows) {
    case 8: rc = launch_scan<8>(a, tiles, threads, smem, stream); break;
    case 16: rc = launch_scan<16>(a, tiles, threads, smem, stream); break;
    case 32: rc = launch_scan<32>(a, tiles, threads, smem, stream); break;
    case 64: rc = launch_scan<64>(a, tiles, threads, smem, stream); break;
  }
  if (rc != 0) return rc;
  bw::launch_pdl(gla_finish_kernel, dim3(n), dim3(128), 0, stream, static_cast<const float*>(o32), u, stride,
                 2 * heads * dim + heads * vdim, norm_w, eps, static_cast<act_t*>(out), heads, vdim);
  return bw::launch_status();
}
