// Routed experts: a token's router scores pick `top` of E small gated feed-forwards.
//
//   z = W_router x (float32, computed by the caller);  s = sigmoid(z)  (or softmax(z))
//   chosen = the `top` largest s, found as the `top` largest z (the lower index wins a tie);  w_k = s_k / (sum of the chosen s + 1e-20) * scale
//   y = sum_k w_k * W_down[e_k] (SiLU(W_gate[e_k] x) * (W_up[e_k] x))
//
// Options: a bias per router output that enters the CHOICE only (chosen = the largest s + bias; the weights stay s);
// experts without a gate, W_down[e] act(W_up[e] x) with the exact GELU; and *identity experts*: router outputs
// from `real` on stand for experts that return their input, so their slots add w_k x and touch no weights.
//
// `route` takes the logits to (expert, weight) pairs, one warp per token.  A (token, k) pair is a *slot*.
// `expert_gate_up` computes the activated hidden row of every slot, `expert_down` its output row, `combine_slots`
// the weighted sum of a token's slots in slot order: no atomics, and a token's result does not depend on the
// batch.  Both read the expert weights as stacked tensors [E, 2 F, K] (gate rows, then up rows) and [E, N, F],
// one warp per output element with 16-byte loads along the reduction (eight on their way per lane), sums in
// float32.  The blocks take the slots in the order of their experts, so slots that share an expert run side by
// side and its rows come from HBM once.  These are the kernels for steps of few tokens and for the 32-bit path.
//
// Steps of more tokens in bfloat16 sort the slots by expert on the device (`sort_slots`: counts, offsets
// padded to whole tiles, the slot list; one block, no host round trip) and run `expert_tiles_*`: 64 slots x
// 64 outputs per block on mma.sync m16n8k16 with float32 accumulators, the expert of a tile found from the
// padded offsets, operands staged through shared memory.  Steps of many tokens sort into tiles of 128 rows,
// copy the tokens' rows into that order and run the package's tcgen05 product in its grouped form twice
// (gate and up with the activation in the epilogue, then down), with a combine in slot order behind it.
#include "common.cuh"

namespace tb {

constexpr int ROUTE_WARPS = 4;

// logits float32 [T, E] -> ids int32 [T, top], weights float32 [T, top].  score: 0 sigmoid, 1 softmax.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
             int T_tokens, int E, int top, int score, int normalize, float scale) {
  extern __shared__ float smem[];  // ROUTE_WARPS * E scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T_tokens) return;
  float* s = smem + warp * E;
  const float* z = logits + (size_t)t * E;
  // Both scores grow with the logit, so the choice is made on the logits: scores that round to the same number
  // (a sigmoid near one) are still told apart.
  float m = -INFINITY, sum = 1.f;
  for (int e = lane; e < E; e += 32) { s[e] = z[e]; m = fmaxf(m, z[e]); }
  if (score == 1) {
    m = warp_max(m);
    sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
    sum = warp_sum(sum);
  }
  // With a bias the choice is made on score + bias instead (the score itself stays the weight).
  if (bias)
    for (int e = lane; e < E; e += 32) s[e] = (score == 1 ? expf(z[e] - m) / sum : 1.f / (1.f + expf(-z[e]))) + bias[e];
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best) { best = s[e]; at = e; }  // ascending e: the lowest index among equals of this lane
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= E) at = 0;  // nothing left to choose from (every score a NaN): no index beyond the row is handed on
    const float zb = bias ? z[at] : best;  // every lane holds the same `at` after the exchange
    const float sc = score == 1 ? expf(zb - m) / sum : 1.f / (1.f + expf(-zb));
    if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      weights[(size_t)t * top + k] = sc;
      s[at] = -INFINITY;
    }
    total += sc;
    __syncwarp();
  }
  if (lane < top) {
    const float w = weights[(size_t)t * top + lane];
    weights[(size_t)t * top + lane] = (normalize ? w / (total + 1e-20f) : w) * scale;
  }
}

template <typename W>
__device__ __forceinline__ float dot_row(const float* xs, const W* row, int K, int lane);

template <>
__device__ __forceinline__ float dot_row<float>(const float* xs, const float* row, int K, int lane) {
  float acc = 0.f;
  if ((K & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int k = lane * 4; k < K; k += 128) {
      const float4 w = *reinterpret_cast<const float4*>(row + k);
      acc = fmaf(xs[k], w.x, acc); acc = fmaf(xs[k + 1], w.y, acc); acc = fmaf(xs[k + 2], w.z, acc); acc = fmaf(xs[k + 3], w.w, acc);
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], row[k], acc);
  }
  return warp_sum(acc);
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* xs, const __nv_bfloat16* row, int K, int lane) {
  float acc = 0.f;
  if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int k0 = lane * 8; k0 < K; k0 += 4 * 256) {  // four 16-byte loads on their way before the first is used
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) raw[u] = k0 + u * 256 < K ? *reinterpret_cast<const uint4*>(row + k0 + u * 256) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 256;
        if (k >= K) break;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc = fmaf(xs[k + 2 * i], f.x, acc);
          acc = fmaf(xs[k + 2 * i + 1], f.y, acc);
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], __bfloat162float(row[k]), acc);
  }
  return warp_sum(acc);
}

// Two rows against the same x at once (a gate row and its up row, or two output rows): eight 16-byte loads are on
// their way per lane before the first is used.  The same sums in the same order as dot_row.
template <typename W>
__device__ __forceinline__ void dot_rows2(const float* xs, const W* r0, const W* r1, int K, int lane, float& d0, float& d1) {
  d0 = dot_row<W>(xs, r0, K, lane);
  d1 = dot_row<W>(xs, r1, K, lane);
}

template <>
__device__ __forceinline__ void dot_rows2<__nv_bfloat16>(const float* xs, const __nv_bfloat16* r0, const __nv_bfloat16* r1, int K,
                                                         int lane, float& d0, float& d1) {
  if ((K & 7) || (reinterpret_cast<uintptr_t>(r0) & 15) || (reinterpret_cast<uintptr_t>(r1) & 15)) {
    d0 = dot_row<__nv_bfloat16>(xs, r0, K, lane);
    d1 = dot_row<__nv_bfloat16>(xs, r1, K, lane);
    return;
  }
  float a0 = 0.f, a1 = 0.f;
  for (int k0 = lane * 8; k0 < K; k0 += 4 * 256) {
    uint4 w0[4], w1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + u * 256;
      w0[u] = k < K ? *reinterpret_cast<const uint4*>(r0 + k) : make_uint4(0, 0, 0, 0);
      w1[u] = k < K ? *reinterpret_cast<const uint4*>(r1 + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + u * 256;
      if (k >= K) break;
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&w0[u]);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&w1[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f0 = __bfloat1622float2(h0[i]), f1 = __bfloat1622float2(h1[i]);
        a0 = fmaf(xs[k + 2 * i], f0.x, a0);
        a0 = fmaf(xs[k + 2 * i + 1], f0.y, a0);
        a1 = fmaf(xs[k + 2 * i], f1.x, a1);
        a1 = fmaf(xs[k + 2 * i + 1], f1.y, a1);
      }
    }
  }
  d0 = warp_sum(a0);
  d1 = warp_sum(a1);
}

constexpr int EX_PER_WARP = 4;  // outputs a warp computes one after the other: x is staged once for 32 of them

// grid (ceil(F / 32), slots): act[slot, j] = SiLU(x_t . gate[e][j]) * (x_t . up[e][j]).
template <typename X, typename W>
__global__ void __launch_bounds__(256)
expert_gate_up_kernel(const X* __restrict__ x, const W* __restrict__ w, const int* __restrict__ ids, const int* __restrict__ order,
                      X* __restrict__ act, int top, int F, int K, int real) {
  extern __shared__ float xs[];  // K floats
  pdl_launch_dependents();
  pdl_wait();
  const int slot = order ? order[blockIdx.y] : blockIdx.y, t = slot / top;  // in `order`, slots of one expert run side by side
  const int e = ids[slot];
  if (e >= real) return;  // an identity expert: the combine takes the token's own row
  const X* xr = x + (size_t)t * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(xr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const W* we = w + (size_t)e * 2 * F * K;
  for (int i = 0; i < EX_PER_WARP; ++i) {
    const int j = (blockIdx.x * EX_PER_WARP + i) * 8 + warp;
    if (j >= F) return;
    float g, u;
    dot_rows2<W>(xs, we + (size_t)j * K, we + (size_t)(F + j) * K, K, lane, g, u);
    if (lane == 0) act[(size_t)slot * F + j] = from_float<X>(g / (1.f + expf(-g)) * u);
  }
}

// Experts named by a table instead of a router: slot (t, k) gets table[token_t][k] and the weight 1 / top.  The host checks
// token ids; an id outside the table, or an entry that names no expert, becomes expert 0 rather than a read or a tile out of range.
__global__ void route_table_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int* __restrict__ ids,
                                   float* __restrict__ weights, long long total, int top, int vocab, int E) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int token = tokens[i / top];
  const int e = (token >= 0 && token < vocab) ? table[(size_t)token * top + (int)(i % top)] : 0;
  ids[i] = (e >= 0 && e < E) ? e : 0;
  weights[i] = 1.f / (float)top;
}

__device__ __forceinline__ float gelu_exact(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }

// The activation of an expert without a gate: 1 the exact GELU, 2 the square of max(v, 0).
__device__ __forceinline__ float plain_act(float v, int act) {
  if (act == 2) { const float r = fmaxf(v, 0.f); return r * r; }
  return gelu_exact(v);
}

// Experts without a gate: act[slot, j] = f(x_t . up[e][j]) with f as `plain_act` names it, up [E, F, K].  grid (ceil(F / 32), slots).
template <typename X, typename W>
__global__ void __launch_bounds__(256)
expert_up_kernel(const X* __restrict__ x, const W* __restrict__ w, const int* __restrict__ ids, const int* __restrict__ order,
                 X* __restrict__ act, int top, int F, int K, int real, int fn) {
  extern __shared__ float xs[];  // K floats
  pdl_launch_dependents();
  pdl_wait();
  const int slot = order ? order[blockIdx.y] : blockIdx.y, t = slot / top;
  const int e = ids[slot];
  if (e >= real) return;
  const X* xr = x + (size_t)t * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(xr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const W* we = w + (size_t)e * F * K;
  for (int i = 0; i < EX_PER_WARP; i += 2) {
    const int j0 = (blockIdx.x * EX_PER_WARP + i) * 8 + warp, j1 = j0 + 8;
    if (j0 >= F) return;
    float d0, d1 = 0.f;
    if (j1 < F) dot_rows2<W>(xs, we + (size_t)j0 * K, we + (size_t)j1 * K, K, lane, d0, d1);
    else d0 = dot_row<W>(xs, we + (size_t)j0 * K, K, lane);
    if (lane == 0) {
      act[(size_t)slot * F + j0] = from_float<X>(plain_act(d0, fn));
      if (j1 < F) act[(size_t)slot * F + j1] = from_float<X>(plain_act(d1, fn));
    }
  }
}

// grid (ceil(N / 32), slots): part[slot, n] = act[slot] . down[e][n]; the combine adds a token's slots in slot order.
template <typename X, typename W>
__global__ void __launch_bounds__(256)
expert_down_kernel(const X* __restrict__ act, const W* __restrict__ w, const int* __restrict__ ids, const int* __restrict__ order,
                   float* __restrict__ part, int N, int F, int real) {
  extern __shared__ float as[];  // F floats
  pdl_launch_dependents();
  pdl_wait();
  const int slot = order ? order[blockIdx.y] : blockIdx.y;
  if (ids[slot] >= real) return;
  for (int i = threadIdx.x; i < F; i += blockDim.x) as[i] = to_float(act[(size_t)slot * F + i]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const W* we = w + (size_t)ids[slot] * N * F;
  for (int i = 0; i < EX_PER_WARP; i += 2) {
    const int n0 = (blockIdx.x * EX_PER_WARP + i) * 8 + warp, n1 = n0 + 8;
    if (n0 >= N) return;
    float d0, d1 = 0.f;
    if (n1 < N) dot_rows2<W>(as, we + (size_t)n0 * F, we + (size_t)n1 * F, F, lane, d0, d1);
    else d0 = dot_row<W>(as, we + (size_t)n0 * F, F, lane);
    if (lane == 0) {
      part[(size_t)slot * N + n0] = d0;
      if (n1 < N) part[(size_t)slot * N + n1] = d1;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Many tokens: slots sorted by expert, tiles on the tensor cores.
constexpr int ET_M = 64, ET_N = 64, ET_K = 32, ET_PAD = 8;

// One block.  counts the slots of each expert, gives expert e the rows [offsets[e], offsets[e + 1]) of the sorted
// list with offsets rounded up to whole tiles of ET_M (rows that pad a tile hold -1), and lists the slots of an
// expert in ascending slot order.  offsets int32 [E + 1]; sorted int32 [capacity], capacity >= slots + E * (ET_M - 1).
// With tile_group (int32 [capacity / tile_rows]) every tile of tile_rows rows also learns its expert (-1: the tile lies
// behind the last expert's rows, or belongs to an identity expert: e >= real), and with position (int32 [slots])
// every slot its row in the sorted list.
__global__ void sort_slots_kernel(const int* __restrict__ ids, int* __restrict__ offsets, int* __restrict__ sorted, int slots,
                                  int E, int capacity, int tile_rows, int* __restrict__ tile_group, int* __restrict__ position,
                                  int real) {
  extern __shared__ int sm[];  // E counts, then E + 1 offsets
  pdl_launch_dependents();
  pdl_wait();
  int* count = sm;
  int* off = sm + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < slots; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = at;
      at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
    }
    off[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) sorted[i] = -1;
  if (tile_group)
    for (int i = threadIdx.x; i < capacity / tile_rows; i += blockDim.x) {
      int e = -1;
      if (i * tile_rows < off[E]) {
        e = 0;
        while (e + 1 < E && off[e + 1] <= i * tile_rows) ++e;
      }
      tile_group[i] = e < real ? e : -1;  // identity experts are the last ones: their tiles are passed over
    }
  __syncthreads();
  // expert by expert, a warp lists its expert's slots in ascending order (ballot + prefix over runs of 32 slots)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int e = warp; e < E; e += nw) {
    int at = off[e];
    for (int base = 0; base < slots; base += 32) {
      const int i = base + lane;
      const bool mine = i < slots && ids[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int row = at + __popc(m & ((1u << lane) - 1u));
        sorted[row] = i;
        if (position) position[i] = row;
      }
      at += __popc(m);
    }
  }
}

__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// A tile of ET_M sorted rows x ET_N outputs of one expert.  MODE 1 (gated): outputs are SiLU(gate) * up for ET_N hidden
// columns (both weight tiles are multiplied), rows are gathered from x by token = slot / top, and the result goes to
// act[sorted position]; MODE 2 (no gate): the same with one weight tile and the activation `fn` (`plain_act`); MODE 0: rows are act[sorted position],
// the result (float32) goes to part[slot].  Tiles of identity experts (e >= real) are passed over.
// 128 threads = 4 warps, warp w owns rows 16 w .. 16 w + 15 of the tile and all ET_N columns.
template <int MODE>
__global__ void __launch_bounds__(128)
expert_tiles_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                    const int* __restrict__ sorted, void* __restrict__ out, int top, int E, int N, int K, int real, int fn) {
  constexpr bool GATED = MODE == 1, GATHER = MODE != 0;
  __shared__ __align__(16) __nv_bfloat16 As[ET_M][ET_K + ET_PAD];
  __shared__ __align__(16) __nv_bfloat16 Bs[GATED ? 2 : 1][ET_N][ET_K + ET_PAD];
  __shared__ int row_src[ET_M];
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = blockIdx.y * ET_M;
  if (row0 >= offsets[E]) return;
  int e = 0;
  while (e + 1 < E && offsets[e + 1] <= row0) ++e;
  if (e >= real) return;
  const int n0 = blockIdx.x * ET_N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < ET_M) {
    const int slot = sorted[row0 + tid];
    row_src[tid] = slot < 0 ? -1 : (GATHER ? slot / top : row0 + tid);
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  float acc[GATED ? 2 : 1][ET_N / 8][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int j = 0; j < ET_N / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][j][i] = 0.f;

  for (int k0 = 0; k0 < K; k0 += ET_K) {
    // 64 rows x 32 columns of 2 bytes = 4 chunks of 16 bytes a row: 256 chunks per operand, two per thread
    for (int c = tid; c < ET_M * 4; c += 128) {
      const int r = c >> 2, kk = (c & 3) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int src = row_src[r];
      if (src >= 0 && k0 + kk < K) v = *reinterpret_cast<const uint4*>(a + (size_t)src * K + k0 + kk);
      *reinterpret_cast<uint4*>(&As[r][kk]) = v;
    }
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
      for (int c = tid; c < ET_N * 4; c += 128) {
        const int r = c >> 2, kk = (c & 3) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n0 + r < N && k0 + kk < K) v = *reinterpret_cast<const uint4*>(we + ((size_t)g * N + n0 + r) * K + k0 + kk);
        *reinterpret_cast<uint4*>(&Bs[g][r][kk]) = v;
      }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < ET_K; ks += 16) {
      uint32_t af[4];
      const int ar = warp * 16 + (lane >> 2), ac = ks + (lane & 3) * 2;
      af[0] = *reinterpret_cast<const uint32_t*>(&As[ar][ac]);
      af[1] = *reinterpret_cast<const uint32_t*>(&As[ar + 8][ac]);
      af[2] = *reinterpret_cast<const uint32_t*>(&As[ar][ac + 8]);
      af[3] = *reinterpret_cast<const uint32_t*>(&As[ar + 8][ac + 8]);
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < ET_N / 8; ++j) {
          uint32_t bf[2];
          const int br = j * 8 + (lane >> 2);
          bf[0] = *reinterpret_cast<const uint32_t*>(&Bs[g][br][ac]);
          bf[1] = *reinterpret_cast<const uint32_t*>(&Bs[g][br][ac + 8]);
          mma_bf16(acc[g][j], af, bf);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < ET_N / 8; ++j)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = warp * 16 + (lane >> 2) + half * 8;
      const int n = n0 + j * 8 + (lane & 3) * 2;
      const int slot = sorted[row0 + r];
      if (slot < 0 || n >= N) continue;
      if (MODE == 2) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)(row0 + r) * N + n;
        o[0] = __float2bfloat16_rn(plain_act(acc[0][j][2 * half], fn));
        if (n + 1 < N) o[1] = __float2bfloat16_rn(plain_act(acc[0][j][2 * half + 1], fn));
      } else if (GATED) {
        const float g0 = acc[0][j][2 * half], g1 = acc[0][j][2 * half + 1];
        const float v0 = g0 / (1.f + expf(-g0)) * acc[GATED ? 1 : 0][j][2 * half];
        const float v1 = g1 / (1.f + expf(-g1)) * acc[GATED ? 1 : 0][j][2 * half + 1];
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)(row0 + r) * N + n;
        o[0] = __float2bfloat16_rn(v0);
        if (n + 1 < N) o[1] = __float2bfloat16_rn(v1);
      } else {
        float* o = reinterpret_cast<float*>(out) + (size_t)slot * N + n;
        o[0] = acc[0][j][2 * half];
        if (n + 1 < N) o[1] = acc[0][j][2 * half + 1];
      }
    }
}

// Rows of x in sorted order: xs[row] = x[sorted[row] / top] (16-byte pieces; K a multiple of 8); rows that pad a tile are zeroed.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted,
                                   __nv_bfloat16* __restrict__ xs, int rows, int K, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = K >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * per_row; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / per_row), c = (int)(i % per_row) << 3;
    const int slot = sorted[row];
    *reinterpret_cast<uint4*>(xs + (size_t)row * K + c) =
        slot < 0 ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(x + (size_t)(slot / top) * K + c);
  }
}

// y[t, n] = sum_k weight[t, k] * part[row of slot t top + k, n], in slot order (position null: the slot's own row).
// A slot of an identity expert (ids given and ids[slot] >= real) adds weight * x[t, n] instead.
template <typename X>
__global__ void combine_slots_kernel(const float* __restrict__ part, const float* __restrict__ weights, float* __restrict__ y,
                                     long long total, int N, int top, const int* __restrict__ position, const int* __restrict__ ids,
                                     int real, const X* __restrict__ x) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / N;
    const int n = (int)(i % N);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      if (ids && ids[t * top + k] >= real) {
        acc = fmaf(weights[t * top + k], to_float(x[i]), acc);
        continue;
      }
      const size_t row = position ? (size_t)position[t * top + k] : (size_t)t * top + k;
      acc = fmaf(weights[t * top + k], part[row * N + n], acc);
    }
    y[i] = acc;
  }
}

}  // namespace tb

extern "C" {

// bias float32 [E] or null: the choice is made on score + bias, the weights are the scores.
int tb_moe_route(void* stream, const float* logits, const float* bias, int* ids, float* weights, int T_tokens, int E, int top,
                 int score, int normalize, float scale) {
  if (T_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > 32 || score < 0 || score > 1) return TB_ERR_BAD_SIZE;
  const size_t smem = (size_t)tb::ROUTE_WARPS * E * sizeof(float);
  if (smem > 48 * 1024) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::route_kernel, dim3((T_tokens + tb::ROUTE_WARPS - 1) / tb::ROUTE_WARPS), dim3(tb::ROUTE_WARPS * 32), smem,
                    stream, logits, bias, ids, weights, T_tokens, E, top, score, normalize, scale);
}

// Routing without a router: ids[t, k] = table[token[t], k], every weight 1 / top.  table int32 [vocab, top].
int tb_moe_route_table(void* stream, const int* tokens, const int* table, int* ids, float* weights, int T_tokens, int top, int vocab,
                       int E) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || vocab <= 0 || E <= 0) return TB_ERR_BAD_SIZE;
  const long long total = (long long)T_tokens * top;
  return tb::launch(tb::route_table_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, stream, tokens, table, ids, weights, total,
                    top, vocab, E);
}

// x [T, K], act [T top, F] of the activations' type `dtype`; the weights of type `dtype` too: w [real, 2 F, K] (gate rows,
// then up rows) with `gated` = 1, else [real, F, K] and an activation without a gate: `gated` = 0 the exact GELU, -1 the square
// of max(v, 0).  Slots whose expert is `real` or more are left out.
// order: int32 [T top] (the slots sorted by expert, so that an expert's rows are fetched once for slots that share it) or null.
int tb_moe_gate_up(void* stream, const void* x, const void* w, const int* ids, const int* order, void* act, int T_tokens, int top,
                   int F, int K, int real, int gated, int dtype) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || F <= 0 || K <= 0 || (long long)T_tokens * top > 65535 || K * sizeof(float) > 48 * 1024) return TB_ERR_BAD_SIZE;
  const dim3 grid((F + 8 * tb::EX_PER_WARP - 1) / (8 * tb::EX_PER_WARP), T_tokens * top);
  if (gated > 0)
    TB_DISPATCH_DTYPE(dtype, tb::launch(tb::expert_gate_up_kernel<T, T>, grid, dim3(256), (size_t)K * sizeof(float), stream,
                                        (const T*)x, (const T*)w, ids, order, (T*)act, top, F, K, real));
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::expert_up_kernel<T, T>, grid, dim3(256), (size_t)K * sizeof(float), stream, (const T*)x,
                                      (const T*)w, ids, order, (T*)act, top, F, K, real, gated < 0 ? 2 : 1));
}

// act [T top, F], w [real, N, F] of type `dtype`; part float32 [T top, N].
int tb_moe_down(void* stream, const void* act, const void* w, const int* ids, const int* order, float* part, int T_tokens, int top,
                int N, int F, int real, int dtype) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || F <= 0 || N <= 0 || (long long)T_tokens * top > 65535 || (size_t)F * sizeof(float) > 48 * 1024) return TB_ERR_BAD_SIZE;
  const dim3 grid((N + 8 * tb::EX_PER_WARP - 1) / (8 * tb::EX_PER_WARP), T_tokens * top);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::expert_down_kernel<T, T>, grid, dim3(256), (size_t)F * sizeof(float), stream, (const T*)act,
                                      (const T*)w, ids, order, part, N, F, real));
}

// The slots sorted by expert, ascending within an expert: order int32 [T top] (offsets int32 [E + 1] is scratch).
int tb_moe_order(void* stream, const int* ids, int* offsets, int* order, int T_tokens, int top, int E) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || E <= 0 || E > 4096) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::sort_slots_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, ids, offsets, order,
                    T_tokens * top, E, T_tokens * top, 1, (int*)nullptr, (int*)nullptr, E);
}

int tb_moe_tile_rows() { return tb::ET_M; }

static int combine(void* stream, const float* part, const float* weights, const int* position, float* y, int T_tokens, int top, int N,
                   const int* ids, int real, const void* x, int x_dtype) {
  const long long total = (long long)T_tokens * N;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  TB_DISPATCH_DTYPE(x_dtype, tb::launch(tb::combine_slots_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, part, weights, y, total, N,
                                        top, position, ids, real, (const T*)x));
}

// The tensor-core path (bfloat16).  offsets int32 [E + 1], sorted int32 [capacity] and act bfloat16 [capacity, F]
// and part float32 [T top, N] are scratch of the caller; capacity = T top + E (tile rows - 1) rounded up to whole tiles.
// E counts every router output; the weights hold the first `real` experts, the others are identity experts.
int tb_moe_tiles(void* stream, const void* x, const void* w_gate_up, const void* w_down, const int* ids, const float* weights,
                 int* offsets, int* sorted, void* act, float* part, float* y, int T_tokens, int top, int E, int N, int F, int K,
                 int capacity, int real, int gated) {
  if (T_tokens <= 0) return 0;
  const int slots = T_tokens * top;
  if (top <= 0 || E <= 0 || E > 4096 || (F & 7) || (K & 7) || N != K || capacity % tb::ET_M || capacity < slots + E * (tb::ET_M - 1))
    return TB_ERR_BAD_SIZE;
  int rc = tb::launch(tb::sort_slots_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, ids, offsets, sorted,
                      slots, E, capacity, (int)tb::ET_M, (int*)nullptr, (int*)nullptr, real);
  if (rc != 0) return rc;
  const int row_tiles = capacity / tb::ET_M;
  const dim3 up_grid((F + tb::ET_N - 1) / tb::ET_N, row_tiles);
  rc = gated > 0 ? tb::launch(tb::expert_tiles_kernel<1>, up_grid, dim3(128), 0, stream, (const __nv_bfloat16*)x,
                              (const __nv_bfloat16*)w_gate_up, offsets, sorted, act, top, E, F, K, real, 0)
                 : tb::launch(tb::expert_tiles_kernel<2>, up_grid, dim3(128), 0, stream, (const __nv_bfloat16*)x,
                              (const __nv_bfloat16*)w_gate_up, offsets, sorted, act, top, E, F, K, real, gated < 0 ? 2 : 1);
  if (rc != 0) return rc;
  rc = tb::launch(tb::expert_tiles_kernel<0>, dim3((N + tb::ET_N - 1) / tb::ET_N, row_tiles), dim3(128), 0, stream,
                  (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, offsets, sorted, part, top, E, N, F, real, 0);
  if (rc != 0) return rc;
  return combine(stream, part, weights, nullptr, y, T_tokens, top, N, real < E ? ids : nullptr, real, x, TB_BF16);
}

// The front and the back of the path that runs the experts as grouped products of 128-row tiles on tcgen05 (the
// package's wide product in its grouped form): `moe_sort_gather` sorts the slots by expert (offsets padded to whole
// tiles), names every tile's expert (-1 for identity experts), remembers every slot's row and copies the tokens' rows
// into sorted order; `moe_combine` adds a token's slots, each from its row, in slot order.  xs bfloat16 [capacity, K];
// capacity a multiple of tile_rows and >= T top + E (tile_rows - 1).
int tb_moe_sort_gather(void* stream, const void* x, const int* ids, int* offsets, int* sorted, int* tile_group, int* position,
                       void* xs, int T_tokens, int top, int E, int K, int capacity, int tile_rows, int real) {
  if (T_tokens <= 0) return 0;
  const int slots = T_tokens * top;
  if (top <= 0 || E <= 0 || E > 4096 || (K & 7) || tile_rows <= 0 || capacity % tile_rows || capacity < slots + E * (tile_rows - 1))
    return TB_ERR_BAD_SIZE;
  int rc = tb::launch(tb::sort_slots_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, ids, offsets, sorted,
                      slots, E, capacity, tile_rows, tile_group, position, real);
  if (rc != 0) return rc;
  long long blocks = ((long long)capacity * (K >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return tb::launch(tb::gather_rows_kernel, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, sorted,
                    (__nv_bfloat16*)xs, capacity, K, top);
}

// ids / real / x (of type x_dtype) only where there are identity experts (ids null: none).
int tb_moe_combine(void* stream, const float* part, const float* weights, const int* position, float* y, int T_tokens, int top, int N,
                   const int* ids, int real, const void* x, int x_dtype) {
  return combine(stream, part, weights, position, y, T_tokens, top, N, ids, real, x, x_dtype);
}

}  // extern "C"
