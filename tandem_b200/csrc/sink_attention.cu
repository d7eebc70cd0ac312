// Windowed attention with kept first tokens, a capped score, a learned bias by distance and a
// softmax sink, over the paged cache; keys and values may have different sizes per head.
//
//   s(i, j) = cap * tanh(scale * (q_i . k_j) / cap) + bias[min(i - j, max_dist)][head]
//   position i sees j  <=>  j <= i and (i - j < window or j < keep_first)        (window 0: all j <= i)
//   o_i = sum_j exp(s(i, j)) v_j / (exp(sink[head]) + sum_j exp(s(i, j)))
//
// Every option is a run-time argument: cap 0 = no cap, bias null = none, sink null = none.  The bias
// table is indexed by distance (the host expands whatever bucketing the model uses into one row per
// distance up to the distance beyond which the bucket no longer changes).
//
// `attention_prepare` (further down) is the step between projection and attention for mixers whose queries and keys are
// convolved over time, normed with a weight and partly rotated; every attention kernel here also takes a gate per
// (token, head) whose sigmoid multiplies the head's output.
//
// Two kernels.  `sink_attention_prep` takes the raw float32 projection [q | k | v] of each token,
// adds the projection biases, divides each q and k head by its root mean square (no weight),
// mixes v with the values another layer made for the same token (v <- (1 - l) v + l v_other), leaves
// q and the unmixed v in place in float32 and writes k and the mixed v to the token's cache slot.
// `sink_attention` then runs one warp per (token, query head) over the visible keys in ascending
// order, 32 keys a turn, scores, softmax statistics and the output accumulator in float32: a
// token's result does not depend on what else is in the batch, bit for bit.  The sink enters as the
// starting state of the online softmax (running maximum = sink, running sum = 1, no value).
#include "cache_layout.cuh"
#include "common.cuh"

namespace tb {

constexpr int SA_MAX_DV = 512;
constexpr int SA_WARPS = 4;

// One warp per (token, unit): units 0..nh-1 are query heads, nh..nh+nkv-1 key heads, then value heads.
template <typename T>
__global__ void __launch_bounds__(128)
sink_attention_prep_kernel(float* __restrict__ qkv, int stride, const float* __restrict__ bias,
                           const float* __restrict__ v_other, int v_other_stride, const float* __restrict__ mix,
                           const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache, int T_tokens, int nh,
                           int nkv, int dk, int dv, int page_size, int unit_norm, float eps, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int units = nh + 2 * nkv;
  const long long g = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (g >= (long long)T_tokens * units) return;
  const int t = (int)(g / units), u = (int)(g % units);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  if (u < nh + nkv) {  // a query or key head: bias, then x / sqrt(mean(x^2) + eps)
    const int col = u * dk;  // q heads, then k heads, lie one behind the other
    float* row = qkv + (size_t)t * stride + col;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) {
      const float x = row[d] + (bias ? bias[col + d] : 0.f);
      ss += x * x;
    }
    ss = warp_sum(ss);
    const float inv = unit_norm ? rsqrtf(ss / (float)dk + eps) : 1.f;
    if (u < nh) {
      for (int d = lane; d < dk; d += 32) row[d] = (row[d] + (bias ? bias[col + d] : 0.f)) * inv;
    } else if (slot >= 0) {
      const int kvh = u - nh;
      T* tile = k_cache + cache_tile(slot / page_size, kvh, nkv, page_size, dk);
      const int r = slot % page_size;
      for (int d = lane; d < dk; d += 32)
        tile[cache_offset<T>(r, d, page_size, dk)] = from_float<T>((row[d] + (bias ? bias[col + d] : 0.f)) * inv);
    }
    return;
  }
  const int kvh = u - nh - nkv;
  const int col = (nh + nkv) * dk + kvh * dv;
  float* row = qkv + (size_t)t * stride + col;
  const float l = v_other ? mix[0] : 0.f;
  T* tile = slot >= 0 ? v_cache + cache_tile(slot / page_size, kvh, nkv, page_size, dv) : nullptr;
  const int r = slot >= 0 ? slot % page_size : 0;
  for (int d = lane; d < dv; d += 32) {
    float x = row[d] + (bias ? bias[col + d] : 0.f);
    row[d] = x;  // the layer's own values, for layers that mix them into theirs
    if (v_other) x = (1.f - l) * x + l * v_other[(size_t)t * v_other_stride + kvh * dv + d];
    if (tile) tile[cache_offset<T>(r, d, page_size, dv)] = from_float<T>(x);
  }
}

// Dot product of the warp's query (shared memory, float32) with one key row of the cache.
template <typename T>
__device__ __forceinline__ float key_dot(const float* qs, const T* tile, int r, int dk, int page_size) {
  float dot = 0.f;
  if (sizeof(T) == 2 && (dk & 7) == 0) {  // eight elements = one 16-byte chunk, whole in either layout
    for (int d = 0; d < dk; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(tile + cache_offset<T>(r, d, page_size, dk));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        dot = fmaf(qs[d + 2 * i], f.x, dot);
        dot = fmaf(qs[d + 2 * i + 1], f.y, dot);
      }
    }
  } else if (sizeof(T) == 4 && (dk & 3) == 0) {
    for (int d = 0; d < dk; d += 4) {
      const float4 f = *reinterpret_cast<const float4*>(tile + cache_offset<T>(r, d, page_size, dk));
      dot = fmaf(qs[d], f.x, dot);
      dot = fmaf(qs[d + 1], f.y, dot);
      dot = fmaf(qs[d + 2], f.z, dot);
      dot = fmaf(qs[d + 3], f.w, dot);
    }
  } else {
    for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], to_float(tile[cache_offset<T>(r, d, page_size, dk)]), dot);
  }
  return dot;
}

// The output gate of a head: sigmoid of one number per (token, head), float32 rows `stride` apart.
__device__ __forceinline__ float head_gate(const float* gate, int stride, int t, int h) {
  return 1.f / (1.f + expf(-gate[(size_t)t * stride + h]));
}

template <typename T>
__global__ void __launch_bounds__(SA_WARPS * 32)
sink_attention_kernel(const float* __restrict__ q, int q_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_of_token,
                      const int* __restrict__ positions, T* __restrict__ out, int T_tokens, int nh, int nkv, int dk, int dv,
                      int page_size, int window, int keep_first, float scale, float cap, const float* __restrict__ bias,
                      int max_dist, const float* __restrict__ sink, const float* __restrict__ gate, int gate_stride) {
  extern __shared__ float smem[];  // SA_WARPS * dk floats: each warp's query
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long g = (long long)blockIdx.x * SA_WARPS + warp;
  if (g >= (long long)T_tokens * nh) return;
  const int t = (int)(g / nh), h = (int)(g % nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  float* qs = smem + warp * dk;
  const float* qrow = q + (size_t)t * q_stride + (size_t)h * dk;
  for (int d = lane; d < dk; d += 32) qs[d] = qrow[d];
  __syncwarp();

  constexpr int MAX_OWN = SA_MAX_DV / 32;  // value dims d = lane + 32 i of this lane
  float acc[MAX_OWN];
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) acc[i] = 0.f;
  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kept = min(keep_first, lo);  // kept first tokens that the window no longer covers
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

  for (int seg = 0; seg < 2; ++seg) {
    const int begin = seg ? lo : 0, end = seg ? pos + 1 : kept;
    for (int base = begin; base < end; base += 32) {
      const int key = base + lane;
      long long tile = -1;  // element offset of the key's (page, kv head) tile, in rows (scaled by the row size where it is used)
      int r_in = 0;
      float s = -INFINITY;
      if (key < end) {
        const int page = table[key / page_size];
        if (page >= 0) {
          tile = (long long)page * nkv + kvh;
          r_in = key % page_size;
          s = key_dot<T>(qs, k_cache + tile * page_size * dk, r_in, dk, page_size) * scale;
          if (cap > 0.f) s = cap * tanhf(s * inv_cap);
          if (bias) s += bias[(size_t)min(pos - key, max_dist) * nh + h];
        }
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
      const float p = (tile >= 0) ? expf(s - m_new) : 0.f;
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < MAX_OWN; ++i) acc[i] *= corr;
      const int count = min(32, end - base);
      for (int j = 0; j < count; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const long long tj = __shfl_sync(0xffffffffu, tile, j);
        const int rin = __shfl_sync(0xffffffffu, r_in, j);
        if (tj < 0) continue;  // the same in every lane
        const T* vr = v_cache + tj * page_size * dv;
#pragma unroll
        for (int i = 0; i < MAX_OWN; ++i) {
          const int d = lane + 32 * i;
          if (d < dv) acc[i] = fmaf(pj, to_float(vr[cache_offset<T>(rin, d, page_size, dv)]), acc[i]);
        }
      }
    }
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate) inv *= head_gate(gate, gate_stride, t, h);
  T* orow = out + (size_t)t * nh * dv + (size_t)h * dv;
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) {
    const int d = lane + 32 * i;
    if (d < dv) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// Decode steps in bfloat16: the keys a token sees are cut into chunks of 128 by absolute position
// (chunk c = keys [128 c, 128 c + 128)), chunk c goes to split c mod `splits`; a block of four warps
// runs one (token, kv head, split) for all query heads of the group (for up to eight of them: larger
// groups are served by several blocks), so a key row is loaded once for the group; a warp takes 32 keys of a chunk (lane = key for the scores, lane = value dims for the
// output).  Every warp keeps the online-softmax state of its keys; the block merges its warps in warp
// order and leaves one partial (maximum, sum, unnormalised output) per (token, head, split); the
// merge kernel adds the splits in split order, the sink first.  Which keys meet in which partial
// depends on the request's own positions only, so a token's result does not depend on the batch.
constexpr int SD_WARPS = 4, SD_CHUNK = 128, SD_MAX_OWN = 8;  // value dims per lane: dv <= 256

template <int GM, typename T>
__global__ void __launch_bounds__(SD_WARPS * 32)
sink_attention_split_kernel(const float* __restrict__ q, int q_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_of_token,
                            const int* __restrict__ positions, float* __restrict__ part_o, float* __restrict__ part_ml, int nh,
                            int nkv, int dk, int dv, int page_size, int window, int keep_first, float scale, float cap,
                            const float* __restrict__ bias, int max_dist) {
  extern __shared__ float smem[];  // GM * dk floats of queries, then SD_WARPS * GM * (2 + dv) floats for the merge
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // more than GM query heads per kv head: blockIdx.y also counts runs of GM heads (each run reads the keys for itself)
  const int runs = (nh / nkv + GM - 1) / GM;
  const int split = blockIdx.x, splits = gridDim.x, kvh = blockIdx.y / runs, h0 = kvh * (nh / nkv) + (blockIdx.y % runs) * GM, t = blockIdx.z;
  const int G = min(GM, (kvh + 1) * (nh / nkv) - h0);  // heads h0 .. h0 + G - 1 are this block's
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kept = min(keep_first, lo);
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  float* q_s = smem;
  float* merge_s = smem + GM * dk;
  for (int i = threadIdx.x; i < G * dk; i += blockDim.x) q_s[i] = q[(size_t)t * q_stride + (size_t)h0 * dk + i];
  __syncthreads();

  float m[GM], l[GM], acc[GM][SD_MAX_OWN];
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < SD_MAX_OWN; ++i) acc[g][i] = 0.f;
  }
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  const int last_chunk = pos / SD_CHUNK, first_window_chunk = lo / SD_CHUNK, kept_chunks = (kept + SD_CHUNK - 1) / SD_CHUNK;
  for (int c = split; c <= last_chunk; c += splits) {
    if (c >= kept_chunks && c < first_window_chunk) {  // between the kept tokens and the window: jump ahead, keeping c = split mod splits
      c += (first_window_chunk - c) / splits * splits;
      if (c < first_window_chunk) continue;
    }
    const int key = c * SD_CHUNK + warp * 32 + lane;
    const bool seen = key <= pos && (key >= lo || key < kept);
    long long tile = -1;
    int r_in = 0;
    float s[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) s[g] = -INFINITY;
    if (seen) {
      const int page = table[key / page_size];
      if (page >= 0) {
        tile = (long long)page * nkv + kvh;
        r_in = key % page_size;
        const T* kr = k_cache + tile * page_size * dk;
        float dot[GM];
#pragma unroll
        for (int g = 0; g < GM; ++g) dot[g] = 0.f;
        if (sizeof(T) == 2 && (dk & 7) == 0) {
          for (int d0 = 0; d0 < dk; d0 += 32) {  // four 16-byte loads are issued before the first is used
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              raw[u] = d0 + 8 * u < dk ? *reinterpret_cast<const uint4*>(kr + cache_offset<T>(r_in, d0 + 8 * u, page_size, dk))
                                       : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int d = d0 + 8 * u;
              if (d >= dk) break;
              const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
              float kf[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(hh[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
#pragma unroll
              for (int g = 0; g < GM; ++g)
                if (g < G) {
                  const float4 q0 = *reinterpret_cast<const float4*>(q_s + g * dk + d), q1 = *reinterpret_cast<const float4*>(q_s + g * dk + d + 4);
                  dot[g] = fmaf(q0.x, kf[0], dot[g]); dot[g] = fmaf(q0.y, kf[1], dot[g]); dot[g] = fmaf(q0.z, kf[2], dot[g]);
                  dot[g] = fmaf(q0.w, kf[3], dot[g]); dot[g] = fmaf(q1.x, kf[4], dot[g]); dot[g] = fmaf(q1.y, kf[5], dot[g]);
                  dot[g] = fmaf(q1.z, kf[6], dot[g]); dot[g] = fmaf(q1.w, kf[7], dot[g]);
                }
            }
          }
        } else {
          for (int d = 0; d < dk; ++d) {
            const float kf = to_float(kr[cache_offset<T>(r_in, d, page_size, dk)]);
#pragma unroll
            for (int g = 0; g < GM; ++g)
              if (g < G) dot[g] = fmaf(q_s[g * dk + d], kf, dot[g]);
          }
        }
#pragma unroll
        for (int g = 0; g < GM; ++g)
          if (g < G) {
            float v = dot[g] * scale;
            if (cap > 0.f) v = cap * tanhf(v * inv_cap);
            if (bias) v += bias[(size_t)min(pos - key, max_dist) * nh + h0 + g];
            s[g] = v;
          }
      }
    }
    float p[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
      p[g] = 0.f;
      if (g < G) {
        const float m_new = fmaxf(m[g], warp_max(s[g]));
        const float corr = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
        p[g] = (tile >= 0) ? expf(s[g] - m_new) : 0.f;
        l[g] = l[g] * corr + warp_sum(p[g]);
        m[g] = m_new;
#pragma unroll
        for (int i = 0; i < SD_MAX_OWN; ++i) acc[g][i] *= corr;
      }
    }
    const unsigned live = __ballot_sync(0xffffffffu, tile >= 0);
    const bool pairs = sizeof(T) == 2 && (dv & 63) == 0;  // a lane owns dims 2 lane + 64 i and the next one: 4-byte loads
    if (live == 0u) continue;
    // keys that are not seen have weight zero and read row 0 of the cache's first tile (always there): no branch in
    // the loop, so that the loads of eight keys are on their way together
    if (pairs) {
      for (int j0 = 0; j0 < 32; j0 += 8) {
        if (!((live >> j0) & 0xffu)) continue;
        __nv_bfloat162 vv[8][SD_MAX_OWN / 2];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {  // the loads of eight keys first
          const long long tj = __shfl_sync(0xffffffffu, tile, j0 + jj);
          const int rin = __shfl_sync(0xffffffffu, r_in, j0 + jj);
          const T* vr = v_cache + (tj < 0 ? 0 : tj) * page_size * dv;
          const int rr = tj < 0 ? 0 : rin;
#pragma unroll
          for (int i = 0; i < SD_MAX_OWN / 2; ++i) {
            const int d = 2 * lane + 64 * i;
            if (d < dv) vv[jj][i] = *reinterpret_cast<const __nv_bfloat162*>(vr + cache_offset<T>(rr, d, page_size, dv));
          }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          float pj[GM];
#pragma unroll
          for (int g = 0; g < GM; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], j0 + jj);
#pragma unroll
          for (int i = 0; i < SD_MAX_OWN / 2; ++i) {
            if (2 * lane + 64 * i < dv) {
              const float2 f = __bfloat1622float2(vv[jj][i]);
#pragma unroll
              for (int g = 0; g < GM; ++g)
                if (g < G) { acc[g][2 * i] = fmaf(pj[g], f.x, acc[g][2 * i]); acc[g][2 * i + 1] = fmaf(pj[g], f.y, acc[g][2 * i + 1]); }
            }
          }
        }
      }
      continue;
    }
#pragma unroll 4
    for (int j = 0; j < 32; ++j) {
      const long long tj = __shfl_sync(0xffffffffu, tile, j);
      const int rin = __shfl_sync(0xffffffffu, r_in, j);
      const T* vr = v_cache + (tj < 0 ? 0 : tj) * page_size * dv;
      const int rr = tj < 0 ? 0 : rin;
      float pj[GM];
#pragma unroll
      for (int g = 0; g < GM; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
      for (int i = 0; i < SD_MAX_OWN; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) {
          const float f = to_float(vr[cache_offset<T>(rr, d, page_size, dv)]);
#pragma unroll
          for (int g = 0; g < GM; ++g)
            if (g < G) acc[g][i] = fmaf(pj[g], f, acc[g][i]);
        }
      }
    }
  }
  // the block's warps in warp order: [warp][g][2 + dv]
  const bool pairs = sizeof(T) == 2 && (dv & 63) == 0;
  const int rec = 2 + dv;
#pragma unroll
  for (int g = 0; g < GM; ++g)
    if (g < G) {
      float* dst = merge_s + ((size_t)warp * GM + g) * rec;
      if (lane == 0) { dst[0] = m[g]; dst[1] = l[g]; }
#pragma unroll
      for (int i = 0; i < SD_MAX_OWN; ++i) {
        const int d = pairs ? 2 * lane + 64 * (i >> 1) + (i & 1) : lane + 32 * i;
        if (d < dv) dst[2 + d] = acc[g][i];
      }
    }
  __syncthreads();
  for (int g = warp; g < G; g += SD_WARPS) {  // warp w merges heads w, w + 4, ...
    float mm = -INFINITY;
    for (int w = 0; w < SD_WARPS; ++w) mm = fmaxf(mm, merge_s[((size_t)w * GM + g) * rec]);
    float ll = 0.f;
    float f[SD_WARPS];
    for (int w = 0; w < SD_WARPS; ++w) {
      const float mw = merge_s[((size_t)w * GM + g) * rec];
      f[w] = mw == -INFINITY ? 0.f : expf(mw - mm);
      ll += merge_s[((size_t)w * GM + g) * rec + 1] * f[w];
    }
    const size_t row = ((size_t)t * nh + h0 + g) * splits + split;
    if (lane == 0) { part_ml[2 * row] = mm; part_ml[2 * row + 1] = ll; }
    for (int d = lane; d < dv; d += 32) {
      float o = 0.f;
      for (int w = 0; w < SD_WARPS; ++w) o += merge_s[((size_t)w * GM + g) * rec + 2 + d] * f[w];
      part_o[row * dv + d] = o;
    }
  }
}

// One warp per (token, head): the sink, then the splits in order.
template <typename T>
__global__ void sink_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            const float* __restrict__ sink, T* __restrict__ out, int rows, int nh, int dv, int splits,
                                            const float* __restrict__ gate, int gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int h = row % nh;
  // lane s reads the statistics of split s (splits <= 32): one round of loads, sums by the warp's fixed butterfly
  const float ms = lane < splits ? part_ml[2 * ((size_t)row * splits + lane)] : -INFINITY;
  const float ls = lane < splits ? part_ml[2 * ((size_t)row * splits + lane) + 1] : 0.f;
  const float mm = fmaxf(sink ? sink[h] : -INFINITY, warp_max(ms));
  const float f = ms == -INFINITY ? 0.f : expf(ms - mm);
  const float ll = warp_sum(ls * f) + (sink ? expf(sink[h] - mm) : 0.f);
  float inv = ll > 0.f ? 1.f / ll : 0.f;
  if (gate) inv *= head_gate(gate, gate_stride, row / nh, h);
  for (int d = lane; d < dv; d += 32) {
    float o = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) o += part_o[((size_t)row * splits + s) * dv + d] * __shfl_sync(0xffffffffu, f, s);
    out[(size_t)row * dv + d] = from_float<T>(o * inv);
  }
}


// ---------------------------------------------------------------------------------------------
// `attention_prepare`: everything between the projection and the attention for mixers whose queries and
// keys are convolved, normed with a weight and rotated.  One block of four warps per token.  The token's
// row of the float32 projection, columns [q: nh dk | k: nkv dk | v: nkv dv] (k and v absent where the
// keys and values are another layer's, v absent where the values are the keys as projected), goes through
//   1. the projection bias, and a causal convolution over time per column, u_t = sum_j w[c, j] x_(t - K + 1 + j):
//      inputs of the same step come from the rows in front, older ones from the request's state (its last
//      K - 1 rows, oldest first; zeroed at admission, which makes the zeros in front of a sequence);
//   2. a norm of q and of k: none; per head without a weight; per head with one weight of dk numbers for all
//      heads; or over the whole of q (of k) with a weight of that size: x / sqrt(mean(x^2) + eps) * w;
//   3. the rotation of the first `rot` numbers of each q and k head, number i paired with i + rot / 2, by the
//      angle position * freq[i] (float32; the host makes the frequency table);
// and leaves q in `q_out` (float32 [T, nh dk]) and k and v in the token's cache slot (a block per token and slice of heads).  The values that go
// into the cache are step 1's, before the norm (also where they are the keys').
struct PrepareArgs {
  const float* proj;
  long long stride;
  const float* bias;   // [columns] or null
  const float* taps;   // [K, columns] (tap j of every column side by side) or null
  int K;
  const float* state;  // rows of state_stride floats: [K - 1, columns]
  long long state_stride;
  const float* q_w;
  const float* k_w;
  int norm;  // 0 none, 1 per head without weight, 2 per head with a shared weight, 3 over all heads with a weight
  float eps;
  const float* freq;  // [rot / 2] or null
  int rot;
  const int* positions;
  const int* seq_of_token;
  const int* seq_starts;
  const int* state_slots;
  const int* slots;
  float* q_out;
  void* k_cache;
  void* v_cache;
  int nh, nkv, dk, dv, page_size;
  int has_kv, v_from_k, write_kv;
};

constexpr int AP_NONE = 0, AP_UNIT = 1, AP_HEAD = 2, AP_WHOLE = 3;
constexpr int AP_THREADS = 256;

// Step 1 for column c of the token in row `row` at position pos: bias and convolution (oldest input first).
__device__ __forceinline__ float prepare_input(const PrepareArgs& a, const float* row, const float* st, int c, int cols, int pos, int start) {
  const float bc = a.bias ? a.bias[c] : 0.f;
  if (!a.taps) return row[c] + bc;
  const int K = a.K;
  float acc = 0.f;
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j, pp = pos - back;
    if (pp < 0) continue;
    const float x = pp >= start ? row[c - (long long)back * a.stride] : st[(size_t)(pp - start + K - 1) * cols + c];
    acc = fmaf(a.taps[(size_t)j * cols + c], x + bc, acc);
  }
  return acc;
}

// grid (tokens, slices): a block of eight warps takes `upb` units of its token, units being the query heads, then the key
// heads (each with its value head where the values are the keys), then the value heads.  A norm over all heads needs the
// sum of squares over the whole of q (of k): every block that has a q (k) unit makes it for itself from global memory, in
// an order that the sizes alone decide, so a token's numbers do not depend on how many slices its step was cut into.
template <typename T>
__global__ void __launch_bounds__(AP_THREADS) attention_prepare_kernel(PrepareArgs a, int upb) {
  extern __shared__ float smem[];  // rot / 2 cosines, rot / 2 sines, then the block's units after step 1
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dk = a.dk, dv = a.dv, half = a.rot / 2;
  const int q_cols = a.nh * dk, k_cols = a.has_kv ? a.nkv * dk : 0;
  const int v_cols = (a.has_kv && !a.v_from_k) ? a.nkv * dv : 0;
  const int cols = q_cols + k_cols + v_cols;
  const int units = a.nh + (a.has_kv ? a.nkv : 0) + (v_cols ? a.nkv : 0);
  const int first = blockIdx.y * upb, last = min(units, first + upb);
  if (first >= units) return;
  const int pos = a.positions[t];
  const float* row = a.proj + (size_t)t * a.stride;
  int start = 0;
  const float* st = nullptr;
  if (a.taps) {
    const int b = a.seq_of_token[t];
    start = a.seq_starts[b];
    if (a.K > 1) st = a.state + (size_t)a.state_slots[b] * a.state_stride;
  }
  float* cs = smem;
  float* sn = smem + half;
  float* u = smem + 2 * half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * a.freq[i], sn + i, cs + i);
  // column of a unit's first number, and the unit's size
  auto unit_col = [&](int unit) { return unit < a.nh + a.nkv ? unit * dk : q_cols + k_cols + (unit - a.nh - a.nkv) * dv; };
  const int c0 = unit_col(first), c1 = last == units ? cols : unit_col(last);
  for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) u[c - c0] = prepare_input(a, row, st, c, cols, pos, start);
  float inv_q = 1.f, inv_k = 1.f;
  if (a.norm == AP_WHOLE) {
    const bool has_q = first < a.nh, has_k = k_cols && last > a.nh && first < a.nh + a.nkv;
    if (has_q) {
      float ss = 0.f;
      for (int c = threadIdx.x; c < q_cols; c += blockDim.x) { const float x = prepare_input(a, row, st, c, cols, pos, start); ss += x * x; }
      inv_q = rsqrtf(block_sum(ss, scratch) / (float)q_cols + a.eps);
    }
    if (has_k) {
      float ss = 0.f;
      for (int c = threadIdx.x; c < k_cols; c += blockDim.x) { const float x = prepare_input(a, row, st, q_cols + c, cols, pos, start); ss += x * x; }
      inv_k = rsqrtf(block_sum(ss, scratch) / (float)k_cols + a.eps);
    }
  }
  __syncthreads();
  const int slot = (a.has_kv && a.write_kv && a.slots) ? a.slots[t] : -1;
  for (int unit = first + warp; unit < last; unit += nwarps) {
    float* x = u + (unit_col(unit) - c0);
    if (unit >= a.nh + a.nkv) {  // a value head of its own
      if (slot < 0) continue;
      const int kvh = unit - a.nh - a.nkv;
      T* tile = reinterpret_cast<T*>(a.v_cache) + cache_tile(slot / a.page_size, kvh, a.nkv, a.page_size, dv);
      const int r = slot % a.page_size;
      for (int d = lane; d < dv; d += 32) tile[cache_offset<T>(r, d, a.page_size, dv)] = from_float<T>(x[d]);
      continue;
    }
    const bool is_q = unit < a.nh;
    const int kvh = unit - a.nh;
    if (!is_q && slot < 0) continue;
    if (!is_q && a.v_from_k) {  // the values are the keys as they stand now
      T* tile = reinterpret_cast<T*>(a.v_cache) + cache_tile(slot / a.page_size, kvh, a.nkv, a.page_size, dv);
      const int r = slot % a.page_size;
      for (int d = lane; d < dv; d += 32) tile[cache_offset<T>(r, d, a.page_size, dv)] = from_float<T>(x[d]);
    }
    if (a.norm != AP_NONE) {
      float inv = is_q ? inv_q : inv_k;
      if (a.norm != AP_WHOLE) {
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss += x[d] * x[d];
        inv = rsqrtf(warp_sum(ss) / (float)dk + a.eps);
      }
      const float* w = is_q ? a.q_w : a.k_w;
      if (a.norm == AP_WHOLE) w += is_q ? unit * dk : kvh * dk;
      const bool weighted = a.norm != AP_UNIT;
      for (int d = lane; d < dk; d += 32) x[d] = x[d] * inv * (weighted ? w[d] : 1.f);
    }
    __syncwarp();
    float* q_dst = is_q ? a.q_out + (size_t)t * q_cols + (size_t)unit * dk : nullptr;
    T* tile = is_q ? nullptr : reinterpret_cast<T*>(a.k_cache) + cache_tile(slot / a.page_size, kvh, a.nkv, a.page_size, dk);
    const int r = is_q ? 0 : slot % a.page_size;
    for (int d = lane; d < dk; d += 32) {
      float y = x[d];
      if (d < a.rot) y = d < half ? x[d] * cs[d] - x[d + half] * sn[d] : x[d] * cs[d - half] + x[d - half] * sn[d - half];
      if (is_q) q_dst[d] = y;
      else tile[cache_offset<T>(r, d, a.page_size, dk)] = from_float<T>(y);
    }
  }
}

// The same for norms that do not reach across heads, sizes that are multiples of four and units of up to 256 numbers: a
// warp per (token, unit), every warp for itself (no meeting of the block); grid (tokens, units / 4).  A lane holds four
// consecutive numbers of every 128 of the unit: 16-byte loads of the inputs, taps, state and weights, 16- or 8-byte
// stores of what the rotation leaves alone.  The rotation goes by pairs through the warp's own piece of shared memory:
// a lane makes the angle of pair p = lane + 32 j once and writes both numbers.  (Counted per unit of 128 numbers, the
// form with one number per lane and turn ran 1,100 instructions and was bound by them, not by its bytes.)
constexpr int AU_GROUPS = 2;

__device__ __forceinline__ float4 prepare_input4(const PrepareArgs& a, const float* row, const float* st, int c, int cols, int pos, int start) {
  const float4 bc = a.bias ? *reinterpret_cast<const float4*>(a.bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  if (!a.taps) {
    const float4 x = *reinterpret_cast<const float4*>(row + c);
    return make_float4(x.x + bc.x, x.y + bc.y, x.z + bc.z, x.w + bc.w);
  }
  const int K = a.K;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < K; ++j) {  // oldest input first
    const int back = K - 1 - j, pp = pos - back;
    if (pp < 0) continue;
    const float* src = pp >= start ? row + c - (long long)back * a.stride : st + (size_t)(pp - start + K - 1) * cols + c;
    const float4 x = *reinterpret_cast<const float4*>(src), w = *reinterpret_cast<const float4*>(a.taps + (size_t)j * cols + c);
    acc.x = fmaf(w.x, x.x + bc.x, acc.x);
    acc.y = fmaf(w.y, x.y + bc.y, acc.y);
    acc.z = fmaf(w.z, x.z + bc.z, acc.z);
    acc.w = fmaf(w.w, x.w + bc.w, acc.w);
  }
  return acc;
}

__device__ __forceinline__ void put4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void put4(__nv_bfloat16* p, const float4& v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
}

// One unit of token t by one warp; x: the warp's own shared memory for the rotation's partners.  inv_q, inv_k: the scales
// of a norm over all heads (made by the caller).
template <typename T>
__device__ __forceinline__ void prepare_unit(const PrepareArgs& a, int t, int unit, float inv_q, float inv_k, float* x, int lane) {
  const int dk = a.dk, dv = a.dv, half = a.rot / 2;
  const int q_cols = a.nh * dk, k_cols = a.has_kv ? a.nkv * dk : 0;
  const int cols = q_cols + k_cols + ((a.has_kv && !a.v_from_k) ? a.nkv * dv : 0);
  const bool is_v = unit >= a.nh + a.nkv, is_q = unit < a.nh;
  const int kvh = is_v ? unit - a.nh - a.nkv : unit - a.nh;
  const int pos = a.positions[t];
  const int slot = (!is_q && a.write_kv && a.slots) ? a.slots[t] : -1;
  const float* row = a.proj + (size_t)t * a.stride;
  int start = 0;
  const float* st = nullptr;
  if (a.taps) {
    const int b = a.seq_of_token[t];
    start = a.seq_starts[b];
    if (a.K > 1) st = a.state + (size_t)a.state_slots[b] * a.state_stride;
  }
  if (!is_q && slot < 0) return;
  const int c0 = is_v ? q_cols + k_cols + kvh * dv : unit * dk, n = is_v ? dv : dk;
  float4 v[AU_GROUPS];
#pragma unroll
  for (int g = 0; g < AU_GROUPS; ++g) {
    const int d = 128 * g + 4 * lane;
    v[g] = d < n ? prepare_input4(a, row, st, c0 + d, cols, pos, start) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int r = slot >= 0 ? slot % a.page_size : 0;
  if (is_v || (!is_q && a.v_from_k)) {  // values of their own, or the keys as they stand now
    T* tile = reinterpret_cast<T*>(a.v_cache) + cache_tile(slot / a.page_size, kvh, a.nkv, a.page_size, dv);
#pragma unroll
    for (int g = 0; g < AU_GROUPS; ++g) {
      const int d = 128 * g + 4 * lane;
      if (d < dv) put4(tile + cache_offset<T>(r, d, a.page_size, dv), v[g]);
    }
    if (is_v) return;
  }
  if (a.norm != AP_NONE) {
    float ss = 0.f;
#pragma unroll
    for (int g = 0; g < AU_GROUPS; ++g) ss += v[g].x * v[g].x + v[g].y * v[g].y + v[g].z * v[g].z + v[g].w * v[g].w;  // zeros beyond the unit
    const float inv = a.norm == AP_WHOLE ? (is_q ? inv_q : inv_k) : rsqrtf(warp_sum(ss) / (float)dk + a.eps);
    const float* w = a.norm == AP_HEAD ? (is_q ? a.q_w : a.k_w) : a.norm == AP_WHOLE ? (is_q ? a.q_w + unit * dk : a.k_w + kvh * dk) : nullptr;
#pragma unroll
    for (int g = 0; g < AU_GROUPS; ++g) {
      const int d = 128 * g + 4 * lane;
      const float4 wv = (w && d < dk) ? *reinterpret_cast<const float4*>(w + d) : make_float4(1.f, 1.f, 1.f, 1.f);
      v[g] = make_float4(v[g].x * inv * wv.x, v[g].y * inv * wv.y, v[g].z * inv * wv.z, v[g].w * inv * wv.w);
    }
  }
  float* q_dst = is_q ? a.q_out + (size_t)t * q_cols + (size_t)unit * dk : nullptr;
  T* tile = is_q ? nullptr : reinterpret_cast<T*>(a.k_cache) + cache_tile(slot / a.page_size, kvh, a.nkv, a.page_size, dk);
  if (half > 0) {
#pragma unroll
    for (int g = 0; g < AU_GROUPS; ++g) {
      const int d = 128 * g + 4 * lane;
      if (d < a.rot) put4(x + d, v[g]);
    }
    __syncwarp();
    for (int p = lane; p < half; p += 32) {
      float sn, cs;
      sincosf((float)pos * a.freq[p], &sn, &cs);
      const float lo = x[p], hi = x[p + half];
      const float y0 = lo * cs - hi * sn, y1 = hi * cs + lo * sn;
      if (is_q) {
        q_dst[p] = y0;
        q_dst[p + half] = y1;
      } else {
        tile[cache_offset<T>(r, p, a.page_size, dk)] = from_float<T>(y0);
        tile[cache_offset<T>(r, p + half, a.page_size, dk)] = from_float<T>(y1);
      }
    }
    __syncwarp();  // the warp's next unit writes x again
  }
#pragma unroll
  for (int g = 0; g < AU_GROUPS; ++g) {
    const int d = 128 * g + 4 * lane;
    if (d >= a.rot && d < dk) {
      if (is_q) put4(q_dst + d, v[g]);
      else put4(tile + cache_offset<T>(r, d, a.page_size, dk), v[g]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attention_prepare_units_kernel(PrepareArgs a, int units, int widest) {
  extern __shared__ __align__(16) float smem[];  // four warps' units
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int unit = blockIdx.y * 4 + warp;
  if (unit >= units) return;
  prepare_unit<T>(a, blockIdx.x, unit, 1.f, 1.f, smem + warp * widest, lane);
}

// With a norm over all heads: grid (tokens, slices of `upb` units), eight warps.  The block makes the sums of squares over
// the whole of q and of k (16-byte loads, a fixed order), then its warps take its units in turn.
template <typename T>
__global__ void __launch_bounds__(AP_THREADS) attention_prepare_whole_kernel(PrepareArgs a, int units, int widest, int upb) {
  extern __shared__ __align__(16) float smem[];  // eight warps' units
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = blockIdx.x;
  const int first = blockIdx.y * upb, last = min(units, first + upb);
  if (first >= units) return;
  const int q_cols = a.nh * a.dk, k_cols = a.has_kv ? a.nkv * a.dk : 0;
  const int cols = q_cols + k_cols + ((a.has_kv && !a.v_from_k) ? a.nkv * a.dv : 0);
  const int pos = a.positions[t];
  const float* row = a.proj + (size_t)t * a.stride;
  int start = 0;
  const float* st = nullptr;
  if (a.taps) {
    const int b = a.seq_of_token[t];
    start = a.seq_starts[b];
    if (a.K > 1) st = a.state + (size_t)a.state_slots[b] * a.state_stride;
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (first < a.nh) {
    float ss = 0.f;
    for (int c = 4 * threadIdx.x; c < q_cols; c += 4 * blockDim.x) {
      const float4 x = prepare_input4(a, row, st, c, cols, pos, start);
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    inv_q = rsqrtf(block_sum(ss, scratch) / (float)q_cols + a.eps);
  }
  if (k_cols && last > a.nh && first < a.nh + a.nkv) {
    float ss = 0.f;
    for (int c = 4 * threadIdx.x; c < k_cols; c += 4 * blockDim.x) {
      const float4 x = prepare_input4(a, row, st, q_cols + c, cols, pos, start);
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    inv_k = rsqrtf(block_sum(ss, scratch) / (float)k_cols + a.eps);
  }
  for (int unit = first + warp; unit < last; unit += blockDim.x >> 5) prepare_unit<T>(a, t, unit, inv_q, inv_k, smem + warp * widest, lane);
}

}  // namespace tb

extern "C" {

// See attention_prepare_kernel.  proj float32 rows `stride` floats apart; bias float32 [columns] or null; taps float32
// [K, columns] or null (then K = 0); state float32 rows of state_stride >= (K - 1) columns floats, indexed by state_slots
// of the token's request (seq_of_token, seq_starts: the tokens a request had before this step); q_w / k_w by `norm`:
// 0 and 1 none, 2 [dk], 3 [nh dk] / [nkv dk]; freq float32 [rot / 2] or null (rot = 0); q_out float32 [T, nh dk];
// caches of the storage type `dtype`.  has_kv 0: the projection has no key or value columns.  v_from_k needs dv == dk.
int tb_attention_prepare(void* stream, const float* proj, long long stride, const float* bias, const float* taps, int K,
                         const float* state, long long state_stride, const float* q_w, const float* k_w, int norm, float eps,
                         const float* freq, int rot, const int* positions, const int* seq_of_token, const int* seq_starts,
                         const int* state_slots, const int* slots, float* q_out, void* k_cache, void* v_cache, int T_tokens, int nh,
                         int nkv, int dk, int dv, int page_size, int has_kv, int v_from_k, int write_kv, int dtype) {
  if (T_tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || norm < 0 || norm > 3 || rot < 0 || rot > dk || (rot & 1) ||
      (rot && !freq) || K < 0 || (K > 0 && !taps) || (K > 1 && !state) || (v_from_k && dv != dk) ||
      (norm >= 2 && (!q_w || (has_kv && !k_w))))
    return TB_ERR_BAD_SIZE;
  const long long cols = (long long)nh * dk + (has_kv ? (long long)nkv * dk + (v_from_k ? 0 : (long long)nkv * dv) : 0);
  if (K > 1 && state_stride < (long long)(K - 1) * cols) return TB_ERR_BAD_SIZE;
  const int units = nh + (has_kv ? nkv : 0) + ((has_kv && !v_from_k) ? nkv : 0);
  // few tokens: a unit per warp and as many blocks as that takes; many tokens: larger slices, fewer blocks that repeat a norm's sums
  int upb = (long long)T_tokens * units <= 8LL * 4 * 148 ? 8 : 16;
  if (norm == 3 && T_tokens > 64) upb = 32;
  const int widest = dk > dv ? dk : dv;
  const size_t smem = ((size_t)rot + (size_t)(upb < units ? upb : units) * widest) * sizeof(float);
  if (smem > 200 * 1024 || (units + upb - 1) / upb > 65535) return TB_ERR_BAD_SIZE;
  tb::PrepareArgs a;
  a.proj = proj; a.stride = stride; a.bias = bias; a.taps = K > 0 ? taps : nullptr; a.K = K; a.state = state; a.state_stride = state_stride;
  a.q_w = q_w; a.k_w = k_w; a.norm = norm; a.eps = eps; a.freq = freq; a.rot = rot; a.positions = positions;
  a.seq_of_token = seq_of_token; a.seq_starts = seq_starts; a.state_slots = state_slots; a.slots = slots; a.q_out = q_out;
  a.k_cache = k_cache; a.v_cache = v_cache; a.nh = nh; a.nkv = nkv; a.dk = dk; a.dv = dv; a.page_size = page_size;
  a.has_kv = has_kv; a.v_from_k = v_from_k; a.write_kv = write_kv;
  if (dtype != TB_F32 && dtype != TB_BF16) return TB_ERR_BAD_DTYPE;
  if (smem > 48 * 1024) {  // per storage type: the attribute belongs to the instantiation
    static size_t allowed[2] = {0, 0};
    if (allowed[dtype] < smem) {
      cudaError_t e = dtype == TB_F32
          ? cudaFuncSetAttribute(tb::attention_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
          : cudaFuncSetAttribute(tb::attention_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      allowed[dtype] = smem;
    }
  }
  const bool fours = !(dk & 3) && !(dv & 3) && !(rot & 3) && !(stride & 3) && !((uintptr_t)proj & 15) && !((uintptr_t)q_out & 15) &&
                     !((uintptr_t)bias & 15) && !((uintptr_t)taps & 15) && !((uintptr_t)state & 15) && !(state_stride & 3) &&
                     !((uintptr_t)q_w & 15) && !((uintptr_t)k_w & 15);
  if (fours && widest <= 128 * tb::AU_GROUPS && (units + 3) / 4 <= 65535) {  // a warp per (token, unit)
    if (norm != 3)
      TB_DISPATCH_DTYPE(dtype, tb::launch(tb::attention_prepare_units_kernel<T>, dim3(T_tokens, (units + 3) / 4), dim3(128),
                                          4 * (size_t)widest * sizeof(float), stream, a, units, widest));
    // few tokens: a unit per warp; many: fewer blocks repeat the sums; a thousand tokens fill the device with one block a token
    const int per_block = (long long)T_tokens * units <= 8LL * 4 * 148 ? 8 : (T_tokens >= 1024 || units <= 24) ? units : 24;
    TB_DISPATCH_DTYPE(dtype, tb::launch(tb::attention_prepare_whole_kernel<T>, dim3(T_tokens, (units + per_block - 1) / per_block),
                                        dim3(tb::AP_THREADS), 8 * (size_t)widest * sizeof(float), stream, a, units, widest, per_block));
  }
  const dim3 grid(T_tokens, (units + upb - 1) / upb);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::attention_prepare_kernel<T>, grid, dim3(tb::AP_THREADS), smem, stream, a, upb));
}

// qkv float32 [T, stride >= nh dk + nkv dk + nkv dv]; bias float32 [nh dk + nkv dk + nkv dv] or null;
// v_other float32 rows of nkv dv values (stride v_other_stride) with mix[0] their share, or null;
// caches of the storage type `dtype`: K [pages, nkv, page_size, dk], V [pages, nkv, page_size, dv].
int tb_sink_attention_prep(void* stream, float* qkv, int stride, const float* bias, const float* v_other, int v_other_stride,
                           const float* mix, const int* slots, void* k_cache, void* v_cache, int T_tokens, int nh, int nkv, int dk,
                           int dv, int page_size, int unit_norm, float eps, int write_kv, int dtype) {
  if (T_tokens <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || (v_other && !mix)) return TB_ERR_BAD_SIZE;
  const long long warps = (long long)T_tokens * (nh + 2 * nkv);
  const int blocks = (int)((warps + 3) / 4);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::sink_attention_prep_kernel<T>, dim3(blocks), dim3(128), 0, stream, qkv, stride, bias, v_other,
                                      v_other_stride, mix, slots, (T*)k_cache, (T*)v_cache, T_tokens, nh, nkv, dk, dv, page_size,
                                      unit_norm, eps, write_kv));
}

// gate: float32 rows of one number per query head (gate_stride floats apart), whose sigmoid multiplies the head's output; or null.
int tb_sink_attention(void* stream, const float* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                      int table_stride, const int* seq_of_token, const int* positions, void* out, int T_tokens, int nh, int nkv,
                      int dk, int dv, int page_size, int window, int keep_first, float scale, float cap, const float* bias,
                      int max_dist, const float* sink, int dtype, const float* gate, int gate_stride) {
  if (T_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dv > tb::SA_MAX_DV || dk > 2048 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || window < 0 ||
      keep_first < 0 || (bias && max_dist < 0))
    return TB_ERR_BAD_SIZE;
  const long long warps = (long long)T_tokens * nh;
  const int blocks = (int)((warps + tb::SA_WARPS - 1) / tb::SA_WARPS);
  const size_t smem = (size_t)tb::SA_WARPS * dk * sizeof(float);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::sink_attention_kernel<T>, dim3(blocks), dim3(tb::SA_WARPS * 32), smem, stream, q, q_stride,
                                      (const T*)k_cache, (const T*)v_cache, block_table, table_stride, seq_of_token, positions,
                                      (T*)out, T_tokens, nh, nkv, dk, dv, page_size, window, keep_first, scale, cap, bias, max_dist,
                                      sink, gate, gate_stride));
}

// The same attention for steps of single tokens, cut over `splits` blocks per (token, kv head):
// part_o float32 [T nh splits dv], part_ml float32 [T nh splits 2] are scratch.  gate as in tb_sink_attention.
int tb_sink_attention_split(void* stream, const float* q, int q_stride, const void* k_cache, const void* v_cache,
                            const int* block_table, int table_stride, const int* seq_of_token, const int* positions, void* out,
                            float* part_o, float* part_ml, int splits, int T_tokens, int nh, int nkv, int dk, int dv, int page_size,
                            int window, int keep_first, float scale, float cap, const float* bias, int max_dist, const float* sink,
                            int dtype, const float* gate, int gate_stride) {
  if (T_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dv > 32 * tb::SD_MAX_OWN || (dk & 3) || nkv <= 0 || nh % nkv != 0 || page_size <= 0 ||
      window < 0 || keep_first < 0 || splits <= 0 || splits > 32 || T_tokens > 65535 || nkv > 65535 || (q_stride & 3) || (bias && max_dist < 0))
    return TB_ERR_BAD_SIZE;
  const int G = nh / nkv, GM = G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : 8;
  const int runs = (G + GM - 1) / GM;  // runs of up to eight query heads per kv head
  const size_t smem = (size_t)(GM * dk + tb::SD_WARPS * GM * (2 + dv)) * sizeof(float);
  if (smem > 48 * 1024 || (long long)nkv * runs > 65535) return TB_ERR_BAD_SIZE;
  const dim3 grid(splits, nkv * runs, T_tokens), block(tb::SD_WARPS * 32);
  int rc = TB_ERR_BAD_DTYPE;
#define TB_SPLIT(GMV, TT)                                                                                                       \
  rc = tb::launch(tb::sink_attention_split_kernel<GMV, TT>, grid, block, smem, stream, q, q_stride, (const TT*)k_cache,          \
                  (const TT*)v_cache, block_table, table_stride, seq_of_token, positions, part_o, part_ml, nh, nkv, dk, dv,      \
                  page_size, window, window > 0 ? keep_first : 0, scale, cap, bias, max_dist)
  if (dtype == TB_BF16) {
    using B = __nv_bfloat16;
    if (GM == 1) TB_SPLIT(1, B); else if (GM == 2) TB_SPLIT(2, B); else if (GM == 4) TB_SPLIT(4, B); else TB_SPLIT(8, B);
  } else if (dtype == TB_F32) {
    if (GM == 1) TB_SPLIT(1, float); else if (GM == 2) TB_SPLIT(2, float); else if (GM == 4) TB_SPLIT(4, float); else TB_SPLIT(8, float);
  }
#undef TB_SPLIT
  if (rc != 0) return rc;
  const int rows = T_tokens * nh;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::sink_attention_merge_kernel<T>, dim3((rows + 3) / 4), dim3(128), 0, stream, part_o, part_ml,
                                      sink, (T*)out, rows, nh, dv, splits, gate, gate_stride));
}

}  // extern "C"
