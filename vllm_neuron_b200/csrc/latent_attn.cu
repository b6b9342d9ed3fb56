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
//     rotated part goes, rotated, to columns [C, C + R) of the head's row of the attention query.
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

}  // extern "C"
