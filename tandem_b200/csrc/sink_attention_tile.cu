// The attention of sink_attention.cu for prompt portions in bfloat16 on the tensor cores: key size
// TB_DK and value size TB_DV fixed at compile time (multiples of 16 up to 128).
//
// The host cuts every request's new tokens into query tiles; one block of four warps runs one tile
// for one kv head.  A tile's 64 rows are (token, query head of the group) pairs, token-major, so one
// pass over the keys serves all the query heads that share the kv head.  Keys and values come from
// the request's pages in stages of 64 keys, 16 bytes per cp.async (a thread per row), two stages in flight; a stage's
// rows keep a padded row-major layout whatever the cache's own tile layout is.  Per stage a warp
// computes S = Q K^T for its 16 rows with mma.sync, then in float32: scale, cap * tanh(s / cap), the
// bias by distance, the mask (causal, window, kept first tokens), the online softmax, whose starting
// state is the sink (running maximum = sink, running sum = 1), and O += P V with P rounded to
// bfloat16.  The keys a tile can see are two runs: the kept first tokens that lie in front of its
// window, and the window of its rows; both are walked in ascending order.
#include "cache_layout.cuh"
#include "common.cuh"
#include "sm100_primitives.cuh"

#if !defined(TB_DK) || !defined(TB_DV)
#error "compile with -DTB_DK=<key size> -DTB_DV=<value size>, multiples of 16"
#endif

namespace tb {

constexpr int DK = TB_DK, DV = TB_DV;
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DV >= 16 && DK <= 128 && DV <= 128, "sizes: multiples of 16 up to 128");
constexpr int ST_WARPS = 4, ST_THREADS = ST_WARPS * 32, ST_BM = ST_WARPS * 16, ST_KEYS = 64;
static_assert(ST_THREADS == 2 * ST_KEYS, "one thread per key row and one per value row of a stage");
constexpr int QP = DK + 8, KP = DK + 8, VP = DV + 8;  // padded rows: ldmatrix without bank conflicts
constexpr int ST_TILE_INTS = 4;                        // first token row, request, first position, number of tokens
constexpr float LOG2E = 1.4426950408889634f;

struct TileArgs {
  const float* q;
  int q_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  int table_stride;
  const int* tiles;
  __nv_bfloat16* out;
  int nh, nkv, page_size, window, keep_first, max_dist;
  float scale, cap;
  const float* bias;
  const float* sink;
  const float* gate;  // one number per (token, query head), rows gate_stride floats apart: its sigmoid multiplies the head's output
  int gate_stride;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Keys [base, base + 64) restricted to [lo, hi) into one stage; rows outside are zeroed (values must
// not be NaN: their weights are zero).  Threads 0..63 bring one key row each, threads 64..127 one value
// row each: one look at the block table and one tile address per row, then its 16-byte pieces.
template <int D, int PITCH>
__device__ __forceinline__ void load_row(const __nv_bfloat16* cache, const int* table, int kvh, int nkv, int ps, int key, bool in_range,
                                         __nv_bfloat16* dst_row) {
  const int page = in_range ? table[key / ps] : -1;
  if (page < 0) {
#pragma unroll
    for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(dst_row + c * 8) = make_uint4(0, 0, 0, 0);
    return;
  }
  const int r = key % ps;
  const __nv_bfloat16* tile = cache + cache_tile(page, kvh, nkv, ps, D);
  if (cache_swizzled<__nv_bfloat16>(D, ps)) {  // [row group][column block][rows of the group][64], chunks XOR-ed with the row
    const int rows = ps < 8 ? ps : 8, group = ps < 8 ? 0 : r >> 3, rr = ps < 8 ? r : r & 7;
#pragma unroll
    for (int c = 0; c < D / 8; ++c)
      cp_async16(dst_row + c * 8, tile + ((group * (D >> 6) + (c >> 3)) * rows + rr) * 64 + (((c & 7) ^ (r & 7)) << 3));
  } else {
#pragma unroll
    for (int c = 0; c < D / 8; ++c) cp_async16(dst_row + c * 8, tile + r * D + c * 8);
  }
}

__device__ __forceinline__ void load_stage(const TileArgs& a, const int* table, int kvh, int base, int lo, int hi,
                                           __nv_bfloat16* ks, __nv_bfloat16* vs, int tid) {
  const int row = tid & (ST_KEYS - 1), key = base + row;
  const bool in_range = key >= lo && key < hi;
  if (tid < ST_KEYS)
    load_row<DK, KP>(a.k_cache, table, kvh, a.nkv, a.page_size, key, in_range, ks + row * KP);
  else
    load_row<DV, VP>(a.v_cache, table, kvh, a.nkv, a.page_size, key, in_range, vs + row * VP);
}

__global__ void __launch_bounds__(ST_THREADS) sink_attention_tile_kernel(const TileArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [ST_BM][QP]
  __nv_bfloat16* k_s = q_s + ST_BM * QP;                             // [2][ST_KEYS][KP]
  __nv_bfloat16* v_s = k_s + 2 * ST_KEYS * KP;                       // [2][ST_KEYS][VP]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = a.tiles + (size_t)blockIdx.x * ST_TILE_INTS;
  const int t0 = tile[0], req = tile[1], p0 = tile[2], ntok = tile[3];
  const int kvh = blockIdx.y, G = a.nh / a.nkv, W = a.window;
  const int* table = a.block_table + (size_t)req * a.table_stride;
  const int kb = W > 0 ? max(0, p0 - W + 1) : 0, ke = p0 + ntok;  // the window of the tile's rows
  const int kept = min(a.keep_first, kb);                          // kept first tokens in front of it
  const int stages_a = (kept + ST_KEYS - 1) / ST_KEYS, stages_b = (ke - kb + ST_KEYS - 1) / ST_KEYS;
  const int num_stages = stages_a + stages_b;

  for (int i = tid; i < ST_BM * (DK / 8); i += ST_THREADS) {  // the query tile: row = token * G + head of the group
    const int row = i / (DK / 8), c = i % (DK / 8);
    const int tl = row / G, g = row % G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tl < ntok) {
      const float* src = a.q + (size_t)(t0 + tl) * a.q_stride + (size_t)(kvh * G + g) * DK + c * 8;
      const float4 f0 = *reinterpret_cast<const float4*>(src), f1 = *reinterpret_cast<const float4*>(src + 4);
      v = make_uint4(pack_bf16(f0.x, f0.y), pack_bf16(f0.z, f0.w), pack_bf16(f1.x, f1.y), pack_bf16(f1.z, f1.w));
    }
    *reinterpret_cast<uint4*>(q_s + row * QP + c * 8) = v;
  }
  auto stage_range = [&](int it, int& base, int& lo, int& hi) {
    if (it < stages_a) { base = it * ST_KEYS; lo = 0; hi = kept; }
    else { base = kb + (it - stages_a) * ST_KEYS; lo = kb; hi = ke; }
  };
  {
    int base, lo, hi;
    stage_range(0, base, lo, hi);
    load_stage(a, table, kvh, base, lo, hi, k_s, v_s, tid);
    cp_async_commit();
  }
  __syncthreads();  // the query tile is written

  int tl_row[2], qpos[2], head[2];  // the two rows this thread holds pieces of: lane / 4 and lane / 4 + 8 of the warp's 16
  float m_run[2], l_run[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + (lane >> 2) + r * 8;
    tl_row[r] = row / G;
    head[r] = kvh * G + row % G;
    qpos[r] = p0 + min(tl_row[r], ntok - 1);  // rows past the last token copy its mask; they are not written
    m_run[r] = a.sink ? a.sink[head[r]] * LOG2E : -INFINITY;  // statistics in units of log2
    l_run[r] = a.sink ? 1.f : 0.f;
  }
  uint32_t qf[DK / 16][4];
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks)
    ldmatrix_x4(qf[ks], smem_u32(q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + ks * 16 + (lane >> 4) * 8));
  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const int warp_first_pos = p0 + min((warp * 16) / G, ntok - 1), warp_last_pos = p0 + min((warp * 16 + 15) / G, ntok - 1);
  const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;

  for (int it = 0; it < num_stages; ++it) {
    const int slot = it & 1;
    if (it + 1 < num_stages) {  // the next stage goes into the other buffer, which everybody left at the end of the last turn
      int base, lo, hi;
      stage_range(it + 1, base, lo, hi);
      load_stage(a, table, kvh, base, lo, hi, k_s + (slot ^ 1) * ST_KEYS * KP, v_s + (slot ^ 1) * ST_KEYS * VP, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    int base, lo, hi;
    stage_range(it, base, lo, hi);
    const __nv_bfloat16* kt = k_s + slot * ST_KEYS * KP;
    const __nv_bfloat16* vt = v_s + slot * ST_KEYS * VP;
    const bool in_window = it >= stages_a;
    // keys of this stage that no row of the warp can see need no arithmetic at all
    const bool skip = in_window && (base > warp_last_pos || (W > 0 && base >= a.keep_first && base + ST_KEYS <= warp_first_pos - W + 1));
    if (!skip) {
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(kt + (sub * 16 + (lane & 7) + (lane >> 4) * 8) * KP + ks * 16 + ((lane >> 3) & 1) * 8));
          mma_bf16_16816(s[2 * sub], qf[ks], b[0], b[1]);
          mma_bf16_16816(s[2 * sub + 1], qf[ks], b[2], b[3]);
        }
      }
      // every key of the stage visible to every row of the warp: no mask to work out
      const bool whole = base >= lo && base + ST_KEYS <= hi && base + ST_KEYS - 1 <= warp_first_pos &&
                         (W <= 0 || base > warp_last_pos - W || base + ST_KEYS <= a.keep_first);
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1, key = base + nt * 8 + (lane & 3) * 2 + (e & 1), q = qpos[r];
          float v = s[nt][e] * a.scale;
          if (a.cap > 0.f) v = a.cap * (1.f - __fdividef(2.f, __expf(2.f * v * inv_cap) + 1.f));  // cap * tanh(v / cap)
          const bool seen = whole || (key >= lo && key < hi && key <= q && (W <= 0 || key > q - W || key < a.keep_first));
          if (seen && a.bias) v += __ldg(a.bias + (size_t)min(q - key, a.max_dist) * a.nh + head[r]);
          v = seen ? v * LOG2E : -INFINITY;
          s[nt][e] = v;
          tile_max[r] = fmaxf(tile_max[r], v);
        }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = tile_max[r];
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
        corr[r] = exp2f(m_run[r] - m_safe);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
        tile_max[r] = m_safe;
      }
      float l_add[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nt][e] = exp2f(s[nt][e] - tile_max[e >> 1]);
          l_add[e >> 1] += s[nt][e];
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {  // the four lanes of a row add up their shares now: the running sum starts at 1 where there is a sink
        l_add[r] += __shfl_xor_sync(0xffffffffu, l_add[r], 1);
        l_add[r] += __shfl_xor_sync(0xffffffffu, l_add[r], 2);
        l_run[r] += l_add[r];
      }
#pragma unroll
      for (int j = 0; j < DV / 8; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t pf[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int j = 0; j < DV / 8; j += 2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + j * 8 + (lane >> 4) * 8));
          mma_bf16_16816(o[j], pf, b[0], b[1]);
          mma_bf16_16816(o[j + 1], pf, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // everybody has left this buffer before the turn after next fills it
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (tl_row[r] >= ntok) continue;
    float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    if (a.gate) inv *= 1.f / (1.f + expf(-a.gate[(size_t)(t0 + tl_row[r]) * a.gate_stride + head[r]]));
    __nv_bfloat16* dst = a.out + (size_t)(t0 + tl_row[r]) * a.nh * DV + (size_t)head[r] * DV + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
  }
}

constexpr size_t tile_smem_bytes() { return (size_t)(ST_BM * QP + 2 * ST_KEYS * KP + 2 * ST_KEYS * VP) * 2; }

}  // namespace tb

extern "C" {

int tb_sink_attention_tile_rows() { return tb::ST_BM; }

// q float32 rows (queries in the first nh * DK columns); tiles [num_tiles, 4] int32 on the device; grid (num_tiles, nkv).
int tb_sink_attention_tile(void* stream, const float* q, int q_stride, const void* k_cache, const void* v_cache,
                           const int* block_table, int table_stride, const int* tiles, int num_tiles, void* out, int nh, int nkv,
                           int page_size, int window, int keep_first, float scale, float cap, const float* bias, int max_dist,
                           const float* sink, const float* gate, int gate_stride) {
  if (num_tiles <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > tb::ST_BM || page_size <= 0 || window < 0 || keep_first < 0 || (q_stride & 3) ||
      (bias && max_dist < 0) || nkv > 65535)
    return TB_ERR_BAD_SIZE;
  tb::TileArgs a;
  a.q = q; a.q_stride = q_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table; a.table_stride = table_stride;
  a.tiles = tiles; a.out = (__nv_bfloat16*)out;
  a.nh = nh; a.nkv = nkv; a.page_size = page_size; a.window = window; a.keep_first = window > 0 ? keep_first : 0; a.max_dist = max_dist;
  a.scale = scale; a.cap = cap; a.bias = bias; a.sink = sink; a.gate = gate; a.gate_stride = gate_stride;
  static bool configured = false;
  const size_t smem = tb::tile_smem_bytes();
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tb::sink_attention_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return tb::launch(tb::sink_attention_tile_kernel, dim3(num_tiles, nkv), dim3(tb::ST_THREADS), smem, stream, a);
}

}  // extern "C"
