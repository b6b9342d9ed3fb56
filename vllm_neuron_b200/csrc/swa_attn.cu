// Sliding-window attention with a softmax sink over the paged KV pools, for layers whose key and value widths differ
// and whose scores carry no positional rotation.
//   * kv_write_vmix: scatters this step's keys and values into the pools by slot; optionally mixes the value with the
//     value the first value-mixing layer produced for the same token, v + lambda (v_first - v), BEFORE it is
//     cached (what is cached is what every later query reads);
//   * swa_sink_attn: ragged batch, one warp per (token, query head).  A query at position i attends keys i - window < j <= i,
//     read through the sequence's block table.  Online softmax in fp32 that STARTS from the sink: running maximum =
//     sink logit, running denominator = 1, accumulator = 0 -- the sink adds exp(sink) to the denominator once, has no key,
//     no value, and is not multiplied by the score scale.
// Pools: K [num_blocks][G][block_size][D], V [num_blocks][G][block_size][Dv] (one (block, kv head) tile is contiguous).
#include <math.h>

#include "hybrid_common.cuh"

namespace b200 {

template <typename KT>
__global__ void kv_write_vmix_kernel(const float* __restrict__ qkv, int ld, int k_col0, int v_col0, float* __restrict__ v_first,
                                     float lam, int mode, KT* __restrict__ k_pool, KT* __restrict__ v_pool,
                                     const int64_t* __restrict__ slots, int G, int D, int Dv, int bs) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / bs, off = slot % bs;
  const float* row = qkv + (int64_t)t * ld;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    stf(k_pool, ((blk * G + g) * bs + off) * D + d, row[k_col0 + i]);
  }
  for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) {
    const int g = i / Dv, d = i - g * Dv;
    float v = row[v_col0 + i];
    if (mode == 1) v_first[(int64_t)t * G * Dv + i] = v;
    if (mode == 2) v = (1.0f - lam) * v + lam * v_first[(int64_t)t * G * Dv + i];
    stf(v_pool, ((blk * G + g) * bs + off) * Dv + d, v);
  }
}

constexpr int ATT_WARPS = 4;

template <typename KT, int MAXC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    swa_sink_attn_kernel(const float* __restrict__ q, int ldq, const KT* __restrict__ k_pool, const KT* __restrict__ v_pool,
                         const int32_t* __restrict__ block_table, int64_t bt_stride, const int32_t* __restrict__ tok_row,
                         const int32_t* __restrict__ tok_pos, const float* __restrict__ sink, float scale, int window,
                         KT* __restrict__ out, int T, int H, int G, int D, int Dv, int bs) {
  griddep_launch();
  griddep_wait();
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * ATT_WARPS + warp;
  if (pair >= (int64_t)T * H) return;
  const int t = (int)(pair / H), h = (int)(pair - (int64_t)t * H);
  const int g = h / (H / G);
  float* qs = qs_all + warp * D;
  for (int d = lane; d < D; d += 32) qs[d] = q[(int64_t)t * ldq + (int64_t)h * D + d];
  __syncwarp();
  const int pos = tok_pos[t];
  const int32_t* bt = block_table + (int64_t)tok_row[t] * bt_stride;
  const int lo = pos - window + 1 > 0 ? pos - window + 1 : 0;
  float m = sink[h], l = 1.0f;  // the sink: exp(sink - m) = 1 in the denominator, nothing in the numerator
  float acc[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc[c] = 0.f;
  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= pos;
    int64_t tile = 0;  // element offset of (block, kv head, token) row 0 in units of one row
    float s = -INFINITY;
    if (valid) {
      const int64_t blk = bt[j / bs];
      tile = (blk * G + g) * bs + (j % bs);
      const KT* kr = k_pool + tile * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot += qs[d] * ldf(kr, d);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[c] *= corr;
    m = m_new;
    const int cnt = pos - j0 + 1 < 32 ? pos - j0 + 1 : 32;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t tj = __shfl_sync(0xffffffffu, tile, jj);
      const KT* vr = v_pool + tj * Dv;
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        const int d = lane + 32 * c;
        if (d < Dv) acc[c] += pj * ldf(vr, d);
      }
    }
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    if (d < Dv) stf(out, ((int64_t)t * H + h) * Dv + d, acc[c] * inv);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_kv_write_vmix(const float* qkv, int ld, int k_col0, int v_col0, float* v_first, float lambda, int mode, void* k_pool,
                       void* v_pool, int kv_dtype, const int64_t* slot_mapping, int T, int G, int D, int Dv, int block_size,
                       void* stream) {
  B200_REQUIRE(qkv && k_pool && v_pool && slot_mapping, "kv_write_vmix: null pointer");
  B200_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || v_first), "kv_write_vmix: mode %d needs the first-layer value buffer", mode);
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(kv_dtype, KT,
                     B200_CUDA_OK(launch_kernel(kv_write_vmix_kernel<KT>, dim3(T), dim3(128), 0, (cudaStream_t)stream, qkv, ld,
                                                k_col0, v_col0, v_first, lambda, mode, (KT*)k_pool, (KT*)v_pool, slot_mapping, G, D,
                                                Dv, block_size)));
  return B200_OK;
}

int b200_swa_sink_attn(const float* q, int ldq, const void* k_pool, const void* v_pool, int kv_dtype, const int32_t* block_table,
                       int64_t bt_stride, const int32_t* tok_row, const int32_t* tok_pos, const float* sink, float scale,
                       int window, void* out, int T, int H, int G, int D, int Dv, int block_size, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && tok_row && tok_pos && sink && out, "swa_sink_attn: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0, "swa_sink_attn: %d query heads over %d kv heads", H, G);
  B200_REQUIRE(window >= 1, "swa_sink_attn: window %d", window);
  B200_REQUIRE(Dv >= 1 && Dv <= 256 && D >= 1 && D <= 1024, "swa_sink_attn: head sizes %d / %d outside 1..1024 / 1..256", D, Dv);
  if (T <= 0) return B200_OK;
  const int64_t pairs = (int64_t)T * H;
  dim3 grid((unsigned)((pairs + ATT_WARPS - 1) / ATT_WARPS));
  const size_t smem = (size_t)ATT_WARPS * D * 4;
  cudaStream_t st = (cudaStream_t)stream;
#define ATT_LAUNCH(MC)                                                                                                      \
  B200_CUDA_OK(launch_kernel(swa_sink_attn_kernel<KT, MC>, grid, dim3(ATT_WARPS * 32), smem, st, q, ldq, (const KT*)k_pool, \
                             (const KT*)v_pool, block_table, bt_stride, tok_row, tok_pos, sink, scale, window, (KT*)out, T, H, G, \
                             D, Dv, block_size))
  B200_DISPATCH_ELEM(kv_dtype, KT, {
    if (Dv <= 64) ATT_LAUNCH(2);
    else if (Dv <= 128) ATT_LAUNCH(4);
    else ATT_LAUNCH(8);
  });
#undef ATT_LAUNCH
  return B200_OK;
}

}  // extern "C"
