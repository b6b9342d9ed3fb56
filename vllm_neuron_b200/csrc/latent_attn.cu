// Latent attention: keys and values of all heads are up-projections of one cached latent c per token, and one rotated
// key part is shared by the heads.  Only [c | k_rot] is cached (one row per token, [num_blocks][block_size][C + R]), and
// attention runs in the latent space: with q' = W_uk^T q_unrotated per head,
//     score = (q' . c + q_rot . k_rot) * scale,      out_latent = sum_j p_j c_j,      value = W_uv out_latent,
// which is multi-query attention with key rows [c | k_rot] (width C + R) and value rows c (the first C columns of the
// same rows): the paged attention kernels of swa_attn.cu / swa_attn_prefill.cu serve it with one kv head, the value pool
// aliased onto the key pool, no sink and no window.  This file holds the per-token steps around them:
//   * latent_kv_write: RMS norm of the latent (plain weight), rotation of the shared key part by the token's position
//     (pairs (2i, 2i + 1) of the first rot_n columns; cos / sin come from a table [positions][rot_n / 2], so any frequency
//     scaling lives in the table), scatter of the row into the pool by slot;
//   * latent_q_prep: per head, the unrotated query part is handed to the absorbing GEMM in the operand type and the
//     rotated part goes, rotated, to columns [C, C + R) of the head's row of the attention query;
//   * latent_attn_decode: single tokens and short portions in bf16 serving on the tensor cores.  All heads of a token read
//     the same cache rows, so the HEADS are the rows of the MMA tile: a CTA takes one token and up to 16 heads, its warps
//     take the visible keys in tiles of 32 round-robin (each warp gathers its tile into its own shared-memory buffer with
//     cp.async, S = Q K^T and O += P V on mma.sync m16n8k16 with the values read from the leading columns of the same
//     tile, fp32 online softmax per warp) and merge through shared memory.
#include <math.h>

#include "hybrid_common.cuh"

namespace b200 {

template <typename KT>
__global__ void latent_kv_write_kernel(const float* __restrict__ in, int ld, int col0, int C, int R, int rot_n,
                                       const float* __restrict__ w, float eps, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int32_t* __restrict__ tok_pos,
                                       const int64_t* __restrict__ slots, KT* __restrict__ pool) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  const float* r = in + (int64_t)t * ld + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) ss += r[i] * r[i];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) red[32] = s;
  }
  __syncthreads();
  if (slot < 0) return;
  const float inv = 1.0f / sqrtf(red[32] / (float)C + eps);
  KT* dst = pool + slot * (C + R);
  for (int i = threadIdx.x; i < C; i += blockDim.x) stf(dst, i, r[i] * inv * w[i]);
  const int half = rot_n >> 1;
  const float* cs = cos_t + (int64_t)tok_pos[t] * half;
  const float* sn = sin_t + (int64_t)tok_pos[t] * half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = r[C + 2 * i], v = r[C + 2 * i + 1];
    stf(dst, C + 2 * i, u * cs[i] - v * sn[i]);
    stf(dst, C + 2 * i + 1, v * cs[i] + u * sn[i]);
  }
  for (int i = rot_n + threadIdx.x; i < R; i += blockDim.x) stf(dst, C + i, r[C + i]);
}

// q fp32 rows [H][D + R] (pitch ldq) -> q_nope [T][H * D] (operand type), q_att[t][h][C .. C + R) = rotated part (fp32)
template <typename OT>
__global__ void latent_q_prep_kernel(const float* __restrict__ q, int ldq, int H, int D, int R, int rot_n, int C,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     const int32_t* __restrict__ tok_pos, OT* __restrict__ q_nope, float* __restrict__ q_att) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const float* r = q + (int64_t)t * ldq;
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
    const int h = i / D, d = i - h * D;
    stf(q_nope, (int64_t)t * H * D + i, r[(int64_t)h * (D + R) + d]);
  }
  const int half = rot_n >> 1;
  const float* cs = cos_t + (int64_t)tok_pos[t] * half;
  const float* sn = sin_t + (int64_t)tok_pos[t] * half;
  float* dst = q_att + (int64_t)t * H * (C + R);
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    const float u = r[(int64_t)h * (D + R) + D + 2 * p], v = r[(int64_t)h * (D + R) + D + 2 * p + 1];
    dst[(int64_t)h * (C + R) + C + 2 * p] = u * cs[p] - v * sn[p];
    dst[(int64_t)h * (C + R) + C + 2 * p + 1] = v * cs[p] + u * sn[p];
  }
  const int rest = R - rot_n;
  for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
    const int h = i / rest, p = rot_n + (i - h * rest);
    dst[(int64_t)h * (C + R) + C + p] = r[(int64_t)h * (D + R) + D + p];
  }
}

constexpr int LD_KEYS = 32;

template <int DV16M>  // accumulator capacity: Dv <= 16 * DV16M
__global__ void __launch_bounds__(256)
    latent_attn_decode_kernel(const float* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ pool,
                              const int32_t* __restrict__ block_table, int64_t bt_stride, const int32_t* __restrict__ tok_row,
                              const int32_t* __restrict__ tok_pos, float scale, __nv_bfloat16* __restrict__ out, int H, int D,
                              int Dv, int bs) {
  griddep_wait();
  extern __shared__ __align__(16) unsigned char la_sm[];
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ldk = D + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(la_sm);                       // [16][ldk]
  __nv_bfloat16* Kt = Qs + 16 * ldk + (size_t)warp * LD_KEYS * ldk;                   // this warp's [32][ldk]
  float* ml = reinterpret_cast<float*>(Qs + 16 * ldk + (size_t)nw * LD_KEYS * ldk);   // [nw][16][2]
  const int t = blockIdx.x, h0 = blockIdx.y * 16;
  const int pos = tok_pos[t];
  const int32_t* bt = block_table + (int64_t)tok_row[t] * bt_stride;
  for (int i = threadIdx.x; i < 16 * (D / 2); i += blockDim.x) {
    const int r = i / (D / 2), d = (i - r * (D / 2)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (h0 + r < H) v = *reinterpret_cast<const float2*>(q + (int64_t)t * ldq + (int64_t)(h0 + r) * D + d);
    *reinterpret_cast<__nv_bfloat162*>(Qs + r * ldk + d) = __floats2bfloat162_rn(v.x, v.y);
  }
  __syncthreads();
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[2 * DV16M][4];
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  const int kch = D / 8;  // 16-byte chunks per cache row
  for (int j0 = LD_KEYS * warp; j0 <= pos; j0 += LD_KEYS * nw) {
    // ---- this warp's 32 cache rows -> its buffer (rows past the token's position are zeros)
    const int jm = j0 + lane;
    const int64_t myrow = jm <= pos ? (int64_t)bt[jm / bs] * bs + (jm % bs) : -1;
    for (int i = lane; i < LD_KEYS * kch; i += 32) {
      const int r = i / kch, c = i - r * kch;
      const int64_t row = __shfl_sync(0xffffffffu, myrow, r);
      cp_async16(smem_u32(Kt + r * ldk + c * 8), pool + (row < 0 ? 0 : row) * D + c * 8, row >= 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    // ---- S = Q K^T: 16 heads x 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
    for (int kk = 0; kk < D; kk += 16) {
      uint32_t af[4];
      ldmatrix_x4(af, smem_u32(Qs + (lane & 15) * ldk + kk + (lane >> 4) * 8));
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        uint32_t bf[4];
        const int mi = lane >> 3;
        ldmatrix_x4(bf, smem_u32(Kt + (16 * jp + (mi >> 1) * 8 + (lane & 7)) * ldk + kk + (mi & 1) * 8));
        mma_bf16_16816(s[2 * jp], af, bf[0], bf[1]);
        mma_bf16_16816(s[2 * jp + 1], af, bf[2], bf[3]);
      }
    }
    // ---- mask (every row of the tile is the same token: one limit), online softmax in fp32
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = j0 + 8 * j + 2 * (lane & 3) + (c & 1);
        const float v = key <= pos ? s[j][c] * scale : -INFINITY;
        s[j][c] = v;
        if (c >= 2) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);  // finite: key j0 is visible
    const float c_lo = __expf(m_lo - mn_lo), c_hi = __expf(m_hi - mn_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
    uint32_t pf[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = __expf(s[j][0] - mn_lo), p1 = __expf(s[j][1] - mn_lo);
      const float p2 = __expf(s[j][2] - mn_hi), p3 = __expf(s[j][3] - mn_hi);
      l_lo += p0 + p1;
      l_hi += p2 + p3;
      pf[j][0] = pack_bf16(p0, p1);
      pf[j][1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int j = 0; j < 2 * DV16M; ++j) {
      o[j][0] *= c_lo;
      o[j][1] *= c_lo;
      o[j][2] *= c_hi;
      o[j][3] *= c_hi;
    }
    // ---- O += P V, the values being the leading Dv columns of the same rows
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint32_t af[4] = {pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1]};
#pragma unroll
      for (int jd = 0; jd < DV16M; ++jd) {
        if (jd * 16 < Dv) {
          uint32_t bf[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(bf, smem_u32(Kt + (16 * ks + (mi & 1) * 8 + (lane & 7)) * ldk + jd * 16 + (mi >> 1) * 8));
          mma_bf16_16816(o[2 * jd], af, bf[0], bf[1]);
          mma_bf16_16816(o[2 * jd + 1], af, bf[2], bf[3]);
        }
      }
    }
    __syncwarp();  // every lane has read the tile before the next one is copied over it
  }
  // the next kernel of the stream may take SM slots from here on: earlier, its waiting CTAs would displace this kernel's own
  griddep_launch();
  // ---- merge the warps: each leaves (m, l, O) in its own buffer
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float* Os = reinterpret_cast<float*>(Kt);  // [16][Dv] fp32 fits: 32 rows of more than Dv bf16
  const int r_lo = lane >> 2;
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j) {
    const int d = 8 * j + 2 * (lane & 3);
    if (d < Dv) {
      Os[r_lo * Dv + d] = o[j][0];
      Os[r_lo * Dv + d + 1] = o[j][1];
      Os[(r_lo + 8) * Dv + d] = o[j][2];
      Os[(r_lo + 8) * Dv + d + 1] = o[j][3];
    }
  }
  if ((lane & 3) == 0) {
    ml[(warp * 16 + r_lo) * 2] = m_lo;
    ml[(warp * 16 + r_lo) * 2 + 1] = l_lo;
    ml[(warp * 16 + r_lo + 8) * 2] = m_hi;
    ml[(warp * 16 + r_lo + 8) * 2 + 1] = l_hi;
  }
  __syncthreads();
  const float* O0 = reinterpret_cast<const float*>(Qs + 16 * ldk);
  const size_t wstride = (size_t)LD_KEYS * ldk / 2;  // floats between two warps' buffers
  for (int i = threadIdx.x; i < 16 * Dv; i += blockDim.x) {
    const int r = i / Dv, d = i - r * Dv;
    if (h0 + r >= H) continue;
    float mt = -INFINITY;
    for (int w = 0; w < nw; ++w) mt = fmaxf(mt, ml[(w * 16 + r) * 2]);
    float lt = 0.f, v = 0.f;
    for (int w = 0; w < nw; ++w) {
      const float f = __expf(ml[(w * 16 + r) * 2] - mt);  // a warp without keys holds m = -inf, l = 0, O = 0
      lt += ml[(w * 16 + r) * 2 + 1] * f;
      v += O0[w * wstride + r * Dv + d] * f;
    }
    out[((int64_t)t * H + h0 + r) * Dv + d] = __float2bfloat16_rn(v / lt);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_latent_kv_write(const float* in, int ld, int col0, int C, int R, int rot_n, const float* norm_w, float eps,
                         const float* cos_table, const float* sin_table, const int32_t* tok_pos, const int64_t* slot_mapping,
                         void* pool, int kv_dtype, int T, void* stream) {
  B200_REQUIRE(in && norm_w && cos_table && sin_table && tok_pos && slot_mapping && pool, "latent_kv_write: null pointer");
  B200_REQUIRE(C >= 1 && R >= 0 && rot_n >= 0 && rot_n <= R && rot_n % 2 == 0, "latent_kv_write: latent %d, rotated part %d of which %d turn",
               C, R, rot_n);
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(kv_dtype, KT,
                     B200_CUDA_OK(launch_kernel(latent_kv_write_kernel<KT>, dim3(T), dim3(128), 0, (cudaStream_t)stream, in, ld, col0,
                                                C, R, rot_n, norm_w, eps, cos_table, sin_table, tok_pos, slot_mapping, (KT*)pool)));
  return B200_OK;
}

int b200_latent_q_prep(const float* q, int ldq, int H, int D, int R, int rot_n, int C, const float* cos_table,
                       const float* sin_table, const int32_t* tok_pos, void* q_nope, int nope_dtype, float* q_att, int T,
                       void* stream) {
  B200_REQUIRE(q && cos_table && sin_table && tok_pos && q_nope && q_att, "latent_q_prep: null pointer");
  B200_REQUIRE(H >= 1 && D >= 1 && rot_n >= 0 && rot_n <= R && rot_n % 2 == 0, "latent_q_prep: bad head shape");
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(nope_dtype, OT,
                     B200_CUDA_OK(launch_kernel(latent_q_prep_kernel<OT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, q, ldq, H, D, R,
                                                rot_n, C, cos_table, sin_table, tok_pos, (OT*)q_nope, q_att)));
  return B200_OK;
}

int b200_latent_attn_decode(const float* q, int ldq, const void* pool, const int32_t* block_table, int64_t bt_stride,
                            const int32_t* tok_row, const int32_t* tok_pos, float scale, void* out, int T, int H, int D, int Dv,
                            int block_size, void* stream) {
  B200_REQUIRE(q && pool && block_table && tok_row && tok_pos && out, "latent_attn_decode: null pointer");
  if (D % 16 || Dv % 16 || Dv > 256 || Dv > D || D > 1024 || (ldq & 1) || ((uintptr_t)q & 7) || H < 1) {
    set_last_error("latent_attn_decode: row width %d / value width %d need multiples of 16 (values <= 256)", D, Dv);
    return B200_ERR_UNSUPPORTED;
  }
  if (T <= 0) return B200_OK;
  int nw = 8;
  auto bytes = [&](int w) { return (size_t)(16 + w * LD_KEYS) * (D + 8) * 2 + (size_t)w * 16 * 2 * 4; };
  while (nw > 1 && bytes(nw) > 200 * 1024) nw >>= 1;
  const size_t smem = bytes(nw);
  dim3 grid(T, (H + 15) / 16);
  typedef __nv_bfloat16 BT;
#define LAD_LAUNCH(M)                                                                                                          \
  do {                                                                                                                         \
    if (smem > 48 * 1024)                                                                                                      \
      B200_CUDA_OK(cudaFuncSetAttribute(latent_attn_decode_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    B200_CUDA_OK(launch_kernel(latent_attn_decode_kernel<M>, grid, dim3(nw * 32), smem, (cudaStream_t)stream, q, ldq,          \
                               (const BT*)pool, block_table, bt_stride, tok_row, tok_pos, scale, (BT*)out, H, D, Dv,          \
                               block_size));                                                                                   \
  } while (0)
  if (Dv <= 64) LAD_LAUNCH(4);
  else if (Dv <= 128) LAD_LAUNCH(8);
  else LAD_LAUNCH(16);
#undef LAD_LAUNCH
  return B200_OK;
}

}  // extern "C"
