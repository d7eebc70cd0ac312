// Sublayers that hang on one float32 stream through a norm on their OUTPUT, and what stands around them:
//
//   grouped RMS norm      a row of W numbers in `groups` equal runs, each divided by sqrt(mean(run^2) + eps),
//                         the whole times a weight                               (`group_norm`: rows gathered, any output type)
//   post-norm add         x <- x + norm(y)                                        (`group_norm_add`)
//   short convolution     h_t = x_t + sum_j w[c, j] x_(t - K + 1 + j), zeros in front of a request; a request's last
//                         K - 1 inputs are its state                              (`short_conv`, `short_conv_state`)
//   depth average         x <- sum_j a_j Y_j over the results Y_0 .. Y_n of the layers so far        (`depth_average`)
//
// and the fused form that a step runs between two sublayers:
//
//   `link`                x' = x + norm(y) [kept as Y_n; x' <- sum_j a_j Y_j], then h = x' + conv(x') in the next
//                         sublayer's input type: the rows' scales first (`row_scales`), then one pass in which a thread
//                         owns a few channels of a run of tokens and keeps the convolution's inputs in registers.
//
// All arithmetic is float32; sums run in an order that depends on nothing but the row, so a token's numbers are the
// same bits however its request is cut into steps or batched.
#include "common.cuh"

namespace tb {

// Pieces of a row: VEC numbers of float32 or bfloat16 into float32 registers and back (VEC 4: one 16- or 8-byte access).
template <int VEC>
__device__ __forceinline__ void load_vec(const float* p, float (&o)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = p[i];
  }
}

template <int VEC>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&o)[VEC]) {
  if constexpr (VEC == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(raw.x << 16); o[1] = __uint_as_float(raw.x & 0xffff0000u);
    o[2] = __uint_as_float(raw.y << 16); o[3] = __uint_as_float(raw.y & 0xffff0000u);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = __bfloat162float(p[i]);
  }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = v[i];
  }
}

template <int VEC>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = __float2bfloat16_rn(v[i]);
  }
}

// Sum of squares of a run of n numbers by one warp (every lane gets it).  A lane takes every 32nd piece of four numbers
// in ascending order into four sums (read in one access where the run starts on a boundary of four, one by one where
// not: a row cut out of a wider array may start anywhere), the numbers behind the last whole piece go to the first
// lanes, and ((s0 + s1) + (s2 + s3)) goes through the warp.  The order depends on n alone, so a row gets the same
// bits from every kernel that norms it, wherever it lies.
template <typename TY>
__device__ __forceinline__ float run_sum_squares(const TY* __restrict__ p, int n, int lane) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const int pieces = n >> 2;
  if ((reinterpret_cast<uintptr_t>(p) & (4 * sizeof(TY) - 1)) == 0) {
#pragma unroll 4
    for (int i = lane; i < pieces; i += 32) {
      float v[4];
      load_vec<4>(p + 4 * i, v);
      s0 = fmaf(v[0], v[0], s0); s1 = fmaf(v[1], v[1], s1); s2 = fmaf(v[2], v[2], s2); s3 = fmaf(v[3], v[3], s3);
    }
  } else {
    for (int i = lane; i < pieces; i += 32) {
      const float v0 = to_float(p[4 * i]), v1 = to_float(p[4 * i + 1]), v2 = to_float(p[4 * i + 2]), v3 = to_float(p[4 * i + 3]);
      s0 = fmaf(v0, v0, s0); s1 = fmaf(v1, v1, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
    }
  }
  if (lane < (n & 3)) { const float v = to_float(p[4 * pieces + lane]); s0 = fmaf(v, v, s0); }
  return warp_sum((s0 + s1) + (s2 + s3));
}

// 1 / sqrt(mean(run^2) + eps) of each run of a row into inv[groups] (shared).  Every thread of the block calls it.
__device__ __forceinline__ void group_scales(const float* __restrict__ row, int W, int groups, float eps, float* inv) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int n = W / groups;
  for (int g = warp; g < groups; g += nw) {
    const float ss = run_sum_squares(row + (size_t)g * n, n, lane);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)n + eps);
  }
}

// inv[t * groups + g] = 1 / sqrt(mean(run g of row t ^2) + eps); one warp per run.
template <typename TY>
__global__ void __launch_bounds__(256)
row_scales_kernel(const TY* __restrict__ y, int W, int groups, float eps, float* __restrict__ inv, long long runs) {
  pdl_launch_dependents();
  pdl_wait();
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= runs) return;
  const int n = W / groups;
  const float ss = run_sum_squares(y + (size_t)r * n, n, threadIdx.x & 31);  // run r of the whole [T, W] array
  if ((threadIdx.x & 31) == 0) inv[r] = 1.f / sqrtf(ss / (float)n + eps);
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

// h[t, c] = x[t, c] + sum_j taps[c, j] * input(t - K + 1 + j), any K.  grid: (tokens, channels / 256).
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ taps, int K, const float* __restrict__ state,
                  long long state_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                  const int* __restrict__ seq_starts, const int* __restrict__ state_slots, T* __restrict__ out, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int b = seq_of_token[t], p = positions[t], start = seq_starts[b];
  const float* st = state ? state + (size_t)state_slots[b] * state_stride : nullptr;
  float acc = x[(size_t)t * W + c];
  for (int j = 0; j < K; ++j) acc = fmaf(taps[(size_t)c * K + j], conv_input(x, W, t, c, p, start, K - 1 - j, st, K), acc);
  out[(size_t)t * W + c] = from_float<T>(acc);
}

// One thread per (request, channel): the request's last K - 1 inputs after this step, oldest first.  An entry that
// still comes from before the step moves down by the number of new tokens; it is read before any turn writes it.
__global__ void short_conv_state_kernel(const float* __restrict__ x, long long x_stride, int W, float* __restrict__ state,
                                        long long state_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                        int requests, int K) {
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
    st[(size_t)k * W + c] = i >= 0 ? x[(size_t)(t0 + i) * x_stride + c] : st[(size_t)(k + n) * W + c];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// The fused link between two sublayers, for rows whose scales `row_scales_kernel` has made.
//   v(t) = x[t] + y[t] * inv[t, group] * weight                            (y null: v(t) = x[t])
//   with planes: kept[t] = v(t);  v(t) <- sum_(j < n) coeff[j] planes[j][t] + coeff[n] v(t)
//   x_out[t] = v(t);  h[t] = v(t) + sum_j taps[c, j] v(t - K + 1 + j)      (inputs in front of the step: the state)
// grid: (runs of `rows` tokens, channels / (256 VEC)).  A thread owns VEC channels and walks down its rows with the last
// K - 1 values of v in registers; at the first row of its run, and wherever another request begins, it makes them anew
// from the rows in front (rows of the same step, so no block waits for another), from the request's state, or as zeros.
// With taps x_out is another buffer than x: other blocks read the x of the rows in front of theirs.
constexpr int LINK_MAX_TAPS = 8;

struct WalkArgs {
  const float* x;
  const void* y;
  const float* inv;
  const float* weight;
  int groups;
  const float* planes;
  long long plane;
  const float* coeff;
  int n_planes;
  float* kept;
  float* x_out;
  const float* taps;
  int K;
  const float* state;
  long long state_stride;
  const int* seq_of_token;
  const int* positions;
  const int* seq_starts;
  const int* state_slots;
  void* h;
  int T, W, rows;
};

template <typename TH, typename TY, int VEC, int KMAX>
__global__ void __launch_bounds__(256, 2)
walk_kernel(const WalkArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * 256 + threadIdx.x) * VEC;
  if (c >= a.W) return;
  const int W = a.W, K = a.taps ? a.K : 0;
  const int r0 = blockIdx.x * a.rows, r1 = min(a.T, r0 + a.rows);
  const TY* y = reinterpret_cast<const TY*>(a.y);
  TH* h = reinterpret_cast<TH*>(a.h);
  const int g = y ? c / (W / a.groups) : 0;
  float wc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) wc[i] = y ? a.weight[c + i] : 0.f;
  float tap[KMAX][VEC];  // tap[back]: the tap on the input `back` tokens in front
#pragma unroll
  for (int back = 0; back < KMAX; ++back)
#pragma unroll
    for (int i = 0; i < VEC; ++i) tap[back][i] = back < K ? a.taps[(size_t)(c + i) * K + (K - 1 - back)] : 0.f;
  const float last = a.planes ? a.coeff[a.n_planes] : 0.f;

  // A row's own numbers come in two halves, so that a thread has the loads of several rows on their way at once.
  auto fetch = [&](int tt, float (&v)[VEC], float (&yv)[VEC], float& s) {
    const size_t at = (size_t)tt * W + c;
    load_vec<VEC>(a.x + at, v);
    if (y) {
      load_vec<VEC>(y + at, yv);
      s = a.inv[(size_t)tt * a.groups + g];
    }
  };
  auto finish = [&](int tt, bool own, float (&v)[VEC], const float (&yv)[VEC], float s) {
    const size_t at = (size_t)tt * W + c;
    if (y) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = fmaf(yv[i] * s, wc[i], v[i]);
    }
    if (a.planes) {
      if (own) store_vec<VEC>(a.kept + at, v);
      float acc[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
      for (int j = 0; j < a.n_planes; ++j) {
        float pv[VEC];
        load_vec<VEC>(a.planes + (size_t)j * a.plane + at, pv);
        const float cj = a.coeff[j];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = fmaf(cj, pv[i], acc[i]);
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = fmaf(last, v[i], acc[i]);
    }
  };
  auto made = [&](int tt, float (&v)[VEC]) {  // a row in front of the run, made again
    float yv[VEC], s = 0.f;
    fetch(tt, v, yv, s);
    finish(tt, false, v, yv, s);
  };

  constexpr int AHEAD = 4;
  float win[KMAX][VEC];  // win[back], back >= 1: the convolution's input `back` tokens in front of the row at hand
  float before[VEC];
  int request = -1;
  // The window of a row where a request begins (within the run: rows of another request in front).
  auto window = [&](int t, int b) {
    const int p = a.positions[t], start = a.seq_starts[b];
    const float* st = a.state + (size_t)a.state_slots[b] * a.state_stride;
#pragma unroll
    for (int back = 1; back < KMAX; ++back) {
      const int q = p - back;
      if (back >= K || q < 0) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) win[back][i] = 0.f;
      } else if (q >= start) {
        made(t - back, win[back]);
      } else {
        load_vec<VEC>(st + (size_t)(q - start + K - 1) * W + c, win[back]);
      }
    }
  };
  if (h && K > 1 && r0 < r1) {  // the run's first row: the same, with every load on its way before the first use
    const int b = a.seq_of_token[r0], p = a.positions[r0], start = a.seq_starts[b];
    const float* st = a.state + (size_t)a.state_slots[b] * a.state_stride;
    float ys[KMAX][VEC], ss[KMAX];
#pragma unroll
    for (int back = 1; back < KMAX; ++back) {
      const int q = p - back;
      if (back >= K || q < 0) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) win[back][i] = 0.f;
      } else if (q >= start) {
        fetch(r0 - back, win[back], ys[back], ss[back]);
      } else {
        load_vec<VEC>(st + (size_t)(q - start + K - 1) * W + c, win[back]);
      }
    }
#pragma unroll
    for (int back = 1; back < KMAX; ++back)
      if (back < K && p - back >= start) finish(r0 - back, false, win[back], ys[back], ss[back]);
    request = b;
  }
  for (int t0 = r0; t0 < r1; t0 += AHEAD) {
    float vs[AHEAD][VEC], ys[AHEAD][VEC], ss[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u)
      if (t0 + u < r1) fetch(t0 + u, vs[u], ys[u], ss[u]);
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int t = t0 + u;
      if (t < r1) {
        float (&v)[VEC] = vs[u];
        finish(t, true, v, ys[u], ss[u]);
        if (a.x_out) store_vec<VEC>(a.x_out + (size_t)t * W + c, v);
        if (h) {
          float acc[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[i] = v[i];
          if (K > 1) {
            const int b = a.seq_of_token[t];
            if (t == r0) {  // made in front of the loop
            } else if (b == request) {  // the row in front is the token in front
#pragma unroll
              for (int back = KMAX - 1; back >= 2; --back)
#pragma unroll
                for (int i = 0; i < VEC; ++i) win[back][i] = win[back - 1][i];
#pragma unroll
              for (int i = 0; i < VEC; ++i) win[1][i] = before[i];
            } else {
              window(t, b);
              request = b;
            }
#pragma unroll
            for (int back = KMAX - 1; back >= 1; --back)  // taps in ascending order, as in short_conv_kernel
#pragma unroll
              for (int i = 0; i < VEC; ++i) acc[i] = back < K ? fmaf(tap[back][i], win[back][i], acc[i]) : acc[i];
          }
          if (K >= 1) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = fmaf(tap[0][i], v[i], acc[i]);
          }
#pragma unroll
          for (int i = 0; i < VEC; ++i) before[i] = v[i];
          store_vec<VEC>(h + (size_t)t * W + c, acc);
        }
      }
    }
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Picks the instance of walk_kernel: four channels per thread where every row, run and buffer starts on 16 bytes
// (bfloat16: 8), registers for 4 or 8 taps.
template <typename TH, typename TY>
static int launch_walk(void* stream, WalkArgs a) {
  const bool wide = a.W % 4 == 0 && (!a.y || (a.W / a.groups) % 4 == 0) && aligned16(a.x) && aligned16(a.y) && aligned16(a.planes) &&
                    a.plane % 4 == 0 && aligned16(a.kept) && aligned16(a.x_out) && aligned16(a.state) && a.state_stride % 4 == 0 &&
                    aligned16(a.h);
  const int vec = wide ? 4 : 1;
  const int gx = (a.W + 256 * vec - 1) / (256 * vec);
  int rows = (int)(((long long)a.T * gx + 148 * 2 - 1) / (148 * 2));  // two blocks fit on a multiprocessor: one wave where 32 rows allow
  rows = rows < 1 ? 1 : (rows > 32 ? 32 : rows);
  if (!a.taps || a.K <= 1) rows = rows < 4 ? rows : 4;  // no rows in front to make again: short runs cost nothing
  a.rows = rows;
  const dim3 grid((a.T + rows - 1) / rows, gx);
  const bool few = !a.taps || a.K <= 4;
  if (wide) return few ? launch(walk_kernel<TH, TY, 4, 4>, grid, dim3(256), 0, stream, a) : launch(walk_kernel<TH, TY, 4, 8>, grid, dim3(256), 0, stream, a);
  return few ? launch(walk_kernel<TH, TY, 1, 4>, grid, dim3(256), 0, stream, a) : launch(walk_kernel<TH, TY, 1, 8>, grid, dim3(256), 0, stream, a);
}

static int launch_walk(void* stream, const WalkArgs& a, int h_dtype, int y_dtype) {
  if (h_dtype == TB_F32) return y_dtype == TB_F32 ? launch_walk<float, float>(stream, a) : launch_walk<float, __nv_bfloat16>(stream, a);
  return y_dtype == TB_F32 ? launch_walk<__nv_bfloat16, float>(stream, a) : launch_walk<__nv_bfloat16, __nv_bfloat16>(stream, a);
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
  if (T_tokens <= 0 || W <= 0) return 0;
  if (K < 0 || (K > 0 && !taps) || (K > 1 && !state)) return TB_ERR_BAD_SIZE;  // K == 0: h = x in the output type
  if (dtype != TB_F32 && dtype != TB_BF16) return TB_ERR_BAD_DTYPE;
  if (K > tb::LINK_MAX_TAPS)
    TB_DISPATCH_DTYPE(dtype, tb::launch(tb::short_conv_kernel<T>, dim3(T_tokens, (W + 255) / 256), dim3(256), 0, stream, x, taps, K, state,
                                        state_stride, seq_of_token, positions, seq_starts, state_slots, (T*)out, W));
  tb::WalkArgs a = {};
  a.x = x; a.groups = 1;
  a.taps = K > 0 ? taps : nullptr; a.K = K; a.state = K > 1 ? state : nullptr; a.state_stride = state_stride;
  a.seq_of_token = seq_of_token; a.positions = positions; a.seq_starts = seq_starts; a.state_slots = state_slots;
  a.h = out; a.T = T_tokens; a.W = W;
  return tb::launch_walk(stream, a, dtype, TB_F32);
}

// x: rows x_stride floats apart, of which the first W columns are the convolution's inputs.
int tb_short_conv_state_rows(void* stream, const float* x, long long x_stride, int W, float* state, long long state_stride,
                             const int* cu_seqlens, const int* state_slots, int requests, int K) {
  if (requests <= 0 || K <= 1) return 0;
  if (x_stride < W) return TB_ERR_BAD_SIZE;
  const long long total = (long long)requests * W;
  return tb::launch(tb::short_conv_state_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, stream, x, x_stride, W, state,
                    state_stride, cu_seqlens, state_slots, requests, K);
}

int tb_short_conv_state(void* stream, const float* x, int W, float* state, long long state_stride, const int* cu_seqlens,
                        const int* state_slots, int requests, int K) {
  return tb_short_conv_state_rows(stream, x, W, W, state, state_stride, cu_seqlens, state_slots, requests, K);
}

// inv [T, groups] = 1 / sqrt(mean(run^2) + eps) of the runs of y's rows (float32 or bfloat16 by y_dtype).
int tb_row_scales(void* stream, const void* y, int y_dtype, int T_tokens, int W, int groups, float eps, float* inv) {
  if (T_tokens <= 0) return 0;
  if (W <= 0 || groups <= 0 || W % groups) return TB_ERR_BAD_SIZE;
  const long long runs = (long long)T_tokens * groups;
  const dim3 grid((unsigned)((runs + 7) / 8));
  if (y_dtype == TB_F32) return tb::launch(tb::row_scales_kernel<float>, grid, dim3(256), 0, stream, (const float*)y, W, groups, eps, inv, runs);
  if (y_dtype == TB_BF16)
    return tb::launch(tb::row_scales_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)y, W, groups, eps, inv, runs);
  return TB_ERR_BAD_DTYPE;
}

// See walk_kernel; inv from tb_row_scales on the same y.  planes null: no depth average (kept unused); taps null: no h.
// With taps x_out must not be x (a block reads the rows in front of its own); without, x_out may be x.
int tb_link(void* stream, const float* x, const void* y, int y_dtype, const float* inv, const float* weight, int groups, const float* planes,
            long long plane, const float* coeff, int n_planes, float* kept, float* x_out, const float* taps, int K, const float* state,
            long long state_stride, const int* seq_of_token, const int* positions, const int* seq_starts, const int* state_slots,
            void* h, int T_tokens, int W, int dtype) {
  if (T_tokens <= 0) return 0;
  if (W <= 0 || groups <= 0 || W % groups || !y || !inv || !x_out || (taps && x_out == x)) return TB_ERR_BAD_SIZE;
  if (taps && (K <= 0 || K > tb::LINK_MAX_TAPS || (K > 1 && !state) || !seq_of_token || !positions || !seq_starts || !state_slots || !h))
    return TB_ERR_BAD_SIZE;
  if (planes && (!coeff || !kept || n_planes < 0)) return TB_ERR_BAD_SIZE;
  if ((dtype != TB_F32 && dtype != TB_BF16) || (y_dtype != TB_F32 && y_dtype != TB_BF16)) return TB_ERR_BAD_DTYPE;
  tb::WalkArgs a = {};
  a.x = x; a.y = y; a.inv = inv; a.weight = weight; a.groups = groups;
  a.planes = planes; a.plane = plane; a.coeff = coeff; a.n_planes = n_planes; a.kept = kept; a.x_out = x_out;
  a.taps = taps; a.K = taps ? K : 0; a.state = (taps && K > 1) ? state : nullptr; a.state_stride = state_stride;
  a.seq_of_token = seq_of_token; a.positions = positions; a.seq_starts = seq_starts; a.state_slots = state_slots;
  a.h = taps ? h : nullptr; a.T = T_tokens; a.W = W;
  return tb::launch_walk(stream, a, dtype, y_dtype);
}

}  // extern "C"
