// Sublayers that hang on one float32 stream through a norm on their OUTPUT, and what stands around them:
//
//   grouped RMS norm      a row of W numbers in `groups` equal runs, each divided by sqrt(mean(run^2) + eps),
//                         the whole times a weight                               (`group_norm`: rows gathered, any output type)
//   post-norm add         x <- x + norm(y)                                        (`group_norm_add`)
//   short convolution     h_t = x_t + sum_j w[c, j] x_(t - K + 1 + j), zeros in front of a request; a request's last
//                         K - 1 inputs are its state                              (`short_conv`, `short_conv_state`)
//   depth average         x <- sum_j a_j Y_j over the results Y_0 .. Y_n of the layers so far        (`depth_average`)
//
// and the two fused forms that a step runs between two sublayers:
//
//   `link`                x' = x + norm(y) [kept as Y_n; x' <- sum_j a_j Y_j], then h = x' + conv(x') in the next
//                         sublayer's input type.  A block owns one token and makes x' for the K - 1 tokens in front of
//                         it again (they are rows of the same step, or the request's state), so no block waits for another.
//
// All arithmetic is float32; sums run in an order that depends on nothing but the row, so a token's numbers are the
// same bits however its request is cut into steps or batched.
#include "common.cuh"

namespace tb {

// 1 / sqrt(mean(run^2) + eps) of each run of a row into inv[groups] (shared).  Every thread of the block calls it.
__device__ __forceinline__ void group_scales(const float* __restrict__ row, int W, int groups, float eps, float* inv) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int n = W / groups;
  for (int g = warp; g < groups; g += nw) {
    const float* p = row + (size_t)g * n;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)n + eps);
  }
}

// out[r] = norm(x[rows ? rows[r] : r]) * weight.  grid: rows.  x rows x_stride floats apart; out [R, W] may be x itself
// (float32, no gather, x_stride == W).
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_kernel(const float* x, long long x_stride, const int* __restrict__ rows, const float* __restrict__ weight, T* out, int W,
                  int groups, float eps) {
  extern __shared__ float inv[];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, t = rows ? rows[r] : r;
  const float* row = x + (size_t)t * x_stride;
  group_scales(row, W, groups, eps, inv);
  __syncthreads();
  const int n = W / groups;
  for (int c = threadIdx.x; c < W; c += blockDim.x) out[(size_t)r * W + c] = from_float<T>(row[c] * inv[c / n] * weight[c]);
}

// residual[t] += norm(y[t]) * weight; with `keep` the new row is also written there.  grid: tokens.
__global__ void __launch_bounds__(256)
group_norm_add_kernel(const float* __restrict__ y, const float* __restrict__ weight, float* __restrict__ residual,
                      float* __restrict__ keep, int W, int groups, float eps) {
  extern __shared__ float inv[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = y + (size_t)t * W;
  group_scales(row, W, groups, eps, inv);
  __syncthreads();
  const int n = W / groups;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = fmaf(row[c] * inv[c / n], weight[c], residual[(size_t)t * W + c]);
    residual[(size_t)t * W + c] = v;
    if (keep) keep[(size_t)t * W + c] = v;
  }
}

// out[i] = sum_j coeff[j] * planes[j * plane + i], j ascending.
__global__ void depth_average_kernel(const float* __restrict__ planes, long long plane, const float* __restrict__ coeff, int n,
                                     float* __restrict__ out, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = fmaf(coeff[j], planes[(size_t)j * plane + i], acc);
    out[i] = acc;
  }
}

// The input of tap j for the token at row t, position p of a request whose rows of this step begin at position `start`:
// a row of this step, the request's state (its last K - 1 inputs before this step, oldest first), or zero.
__device__ __forceinline__ float conv_input(const float* __restrict__ x, int W, int t, int c, int p, int start, int back,
                                            const float* __restrict__ st, int K) {
  const int q = p - back;
  if (q < 0) return 0.f;
  if (q >= start) return x[(size_t)(t - back) * W + c];
  return st[(size_t)(q - start + K - 1) * W + c];
}

// h[t, c] = x[t, c] + sum_j taps[c, j] * input(t - K + 1 + j).  One thread per (token, channel).
template <typename T>
__global__ void short_conv_kernel(const float* __restrict__ x, const float* __restrict__ taps, int K, const float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                  const int* __restrict__ seq_starts, const int* __restrict__ state_slots, T* __restrict__ out,
                                  long long total, int W) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / W), c = (int)(i % W);
    const int b = seq_of_token[t], p = positions[t], start = seq_starts[b];
    const float* st = state ? state + (size_t)state_slots[b] * state_stride : nullptr;
    float acc = x[i];
    for (int j = 0; j < K; ++j) acc = fmaf(taps[(size_t)c * K + j], conv_input(x, W, t, c, p, start, K - 1 - j, st, K), acc);
    out[i] = from_float<T>(acc);
  }
}

// One thread per (request, channel): the request's last K - 1 inputs after this step, oldest first.  An entry that
// still comes from before the step moves down by the number of new tokens; it is read before any turn writes it.
__global__ void short_conv_state_kernel(const float* __restrict__ x, int W, float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int requests, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)requests * W) return;
  const int b = (int)(idx / W), c = (int)(idx % W);
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[b] * state_stride;
  for (int k = 0; k < K - 1; ++k) {
    const int i = n - (K - 1) + k;
    st[(size_t)k * W + c] = i >= 0 ? x[(size_t)(t0 + i) * W + c] : st[(size_t)(k + n) * W + c];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// The fused link between two sublayers.  grid: tokens; dynamic shared memory: K * groups floats.
//   v(tt) = x[tt] + norm(y[tt]) * weight                                   for tt = t - K + 1 .. t within this step
//   with planes: kept[t] = v(t);  v(tt) <- sum_(j < n) coeff[j] planes[j][tt] + coeff[n] v(tt)
//   x_out[t] = v(t);  h[t] = v(t) + sum_j taps[c, j] v(t - K + 1 + j)      (inputs in front of the step: the state)
// With taps x_out is another buffer than x: the blocks of later tokens read x[t].  taps null: no h is made, and x_out may be x.
constexpr int LINK_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
link_kernel(const float* x, const float* __restrict__ y, const float* __restrict__ weight, int groups, float eps,
            const float* __restrict__ planes, long long plane, const float* __restrict__ coeff, int n_planes, float* __restrict__ kept,
            float* x_out, const float* __restrict__ taps, int K, const float* __restrict__ state, long long state_stride,
            const int* __restrict__ seq_of_token, const int* __restrict__ positions, const int* __restrict__ seq_starts,
            const int* __restrict__ state_slots, T* __restrict__ h, int W) {
  extern __shared__ float inv[];  // [K][groups]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int b = 0, p = 0, start = 0;  // the batch arrays are only there (and only needed) with a convolution
  if (taps) { b = seq_of_token[t]; p = positions[t]; start = seq_starts[b]; }
  const int reach = taps ? min(K - 1, p - start) : 0;  // tokens in front of t that are rows of this step
  for (int back = 0; back <= reach; ++back) group_scales(y + (size_t)(t - back) * W, W, groups, eps, inv + back * groups);
  __syncthreads();
  const int n = W / groups;
  const float* st = (taps && state) ? state + (size_t)state_slots[b] * state_stride : nullptr;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float wc = weight[c];
    float v[LINK_MAX_TAPS];
#pragma unroll
    for (int back = 0; back < LINK_MAX_TAPS; ++back) {
      if (back > reach) break;
      const size_t at = (size_t)(t - back) * W + c;
      float made = fmaf(y[at] * inv[back * groups + c / n], wc, x[at]);
      if (planes) {
        if (back == 0) kept[at] = made;
        float acc = 0.f;
        for (int j = 0; j < n_planes; ++j) acc = fmaf(coeff[j], planes[(size_t)j * plane + at], acc);
        made = fmaf(coeff[n_planes], made, acc);
      }
      v[back] = made;
    }
    x_out[(size_t)t * W + c] = v[0];
    if (!taps) continue;
    float acc = v[0];
#pragma unroll
    for (int back = LINK_MAX_TAPS - 1; back >= 0; --back) {  // tap j = K - 1 - back, ascending as in short_conv_kernel
      if (back >= K) continue;
      const int q = p - back;
      float in = 0.f;
      if (q >= start) in = v[back];
      else if (q >= 0) in = st[(size_t)(q - start + K - 1) * W + c];
      acc = fmaf(taps[(size_t)c * K + (K - 1 - back)], in, acc);
    }
    h[(size_t)t * W + c] = from_float<T>(acc);
  }
}

}  // namespace tb

extern "C" {

static int flat_blocks(long long total) {
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

// out [R, W] of type `dtype` = norm(x[rows[r]]) * weight; rows null: row r itself.  x float32 rows of W numbers, x_stride apart.
int tb_group_norm(void* stream, const float* x, long long x_stride, const int* rows, const float* weight, void* out, int R, int W,
                  int groups, float eps, int dtype) {
  if (R <= 0) return 0;
  if (W <= 0 || groups <= 0 || W % groups || groups > 4096) return TB_ERR_BAD_SIZE;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::group_norm_kernel<T>, dim3(R), dim3(256), (size_t)groups * sizeof(float), stream, x, x_stride,
                                      rows, weight, (T*)out, W, groups, eps));
}

int tb_group_norm_add(void* stream, const float* y, const float* weight, float* residual, float* keep, int T_tokens, int W,
                      int groups, float eps) {
  if (T_tokens <= 0) return 0;
  if (W <= 0 || groups <= 0 || W % groups || groups > 4096) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::group_norm_add_kernel, dim3(T_tokens), dim3(256), (size_t)groups * sizeof(float), stream, y, weight, residual,
                    keep, W, groups, eps);
}

int tb_depth_average(void* stream, const float* planes, long long plane, const float* coeff, int n, float* out, long long total) {
  if (total <= 0) return 0;
  if (n <= 0) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::depth_average_kernel, dim3(flat_blocks(total)), dim3(256), 0, stream, planes, plane, coeff, n, out, total);
}

// h [T, W] of type `dtype` = x + conv(x); taps float32 [W, K]; state float32 rows of state_stride floats, a request's
// last K - 1 inputs [K - 1, W] at the row's start (null where K == 1).
int tb_short_conv(void* stream, const float* x, const float* taps, int K, const float* state, long long state_stride,
                  const int* seq_of_token, const int* positions, const int* seq_starts, const int* state_slots, void* out, int T_tokens,
                  int W, int dtype) {
  const long long total = (long long)T_tokens * W;
  if (total <= 0) return 0;
  if (K < 0 || (K > 0 && !taps) || (K > 1 && !state)) return TB_ERR_BAD_SIZE;  // K == 0: h = x in the output type
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::short_conv_kernel<T>, dim3(flat_blocks(total)), dim3(256), 0, stream, x, taps, K, state,
                                      state_stride, seq_of_token, positions, seq_starts, state_slots, (T*)out, total, W));
}

int tb_short_conv_state(void* stream, const float* x, int W, float* state, long long state_stride, const int* cu_seqlens,
                        const int* state_slots, int requests, int K) {
  if (requests <= 0 || K <= 1) return 0;
  const long long total = (long long)requests * W;
  return tb::launch(tb::short_conv_state_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, stream, x, W, state, state_stride,
                    cu_seqlens, state_slots, requests, K);
}

// See link_kernel.  planes null: no depth average (kept unused); taps null: no h.  With taps x_out must not be x (a block
// reads the rows in front of its own); without, a block reads its own row only and x_out may be x.
int tb_link(void* stream, const float* x, const float* y, const float* weight, int groups, float eps, const float* planes,
            long long plane, const float* coeff, int n_planes, float* kept, float* x_out, const float* taps, int K, const float* state,
            long long state_stride, const int* seq_of_token, const int* positions, const int* seq_starts, const int* state_slots,
            void* h, int T_tokens, int W, int dtype) {
  if (T_tokens <= 0) return 0;
  if (W <= 0 || groups <= 0 || W % groups || (taps && x_out == x)) return TB_ERR_BAD_SIZE;
  if (taps && (K <= 0 || K > tb::LINK_MAX_TAPS || (K > 1 && !state) || !seq_of_token || !positions || !seq_starts || !state_slots || !h))
    return TB_ERR_BAD_SIZE;
  if (planes && (!coeff || !kept || n_planes < 0)) return TB_ERR_BAD_SIZE;
  const int kk = taps ? K : 1;
  const size_t smem = (size_t)kk * groups * sizeof(float);
  if (smem > 48 * 1024) return TB_ERR_BAD_SIZE;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::link_kernel<T>, dim3(T_tokens), dim3(256), smem, stream, x, y, weight, groups, eps, planes,
                                      plane, coeff, n_planes, kept, x_out, taps, kk, state, state_stride, seq_of_token, positions,
                                      seq_starts, state_slots, (T*)h, W));
}

}  // extern "C"
