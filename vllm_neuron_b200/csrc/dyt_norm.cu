// Elementwise and per-row kernels of the hybrid decoder: scaled embedding gather into the fp32 residual stream,
// Dynamic-Tanh norm (gain * tanh(a x) + shift, elementwise, no row statistics), the fused "residual += norm(branch); next = norm(residual)"
// step, the gated grouped RMS norm that closes a state-space mixer, and the clamped gated-linear-unit activation.
// The residual stream and all norm arithmetic are fp32; outputs that feed a GEMM are written in the GEMM operand type.
#include "hybrid_common.cuh"

namespace b200 {

template <typename WT>
__global__ void embed_scale_kernel(const int32_t* __restrict__ tokens, const WT* __restrict__ table, float* __restrict__ out,
                                   int W, int V, float scale) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(int64_t)t * W + i] = ldf(table, (int64_t)tok * W + i) * scale;
}

template <typename OT>
__global__ void dyt_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float alpha,
                           OT* __restrict__ out, int W, int64_t total) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % W);
    stf(out, i, tanhf(alpha * x[i]) * w[c] + b[c]);
  }
}

// x[t] += dyt1( sum_{c < nsum} y[(t * nsum + c)] + y2[t] );   out2[t] = dyt2(x[t])  (when out2 is given)
template <typename OT>
__global__ void dyt_residual_kernel(float* __restrict__ x, const float* __restrict__ y, int nsum, const float* __restrict__ y2,
                                    const float* __restrict__ w1, const float* __restrict__ b1, float a1,
                                    const float* __restrict__ w2, const float* __restrict__ b2, float a2, OT* __restrict__ out2,
                                    int W, int64_t total) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / W;
    const int c = (int)(i - t * W);
    float s = 0.f;
    for (int k = 0; k < nsum; ++k) s += y[(t * nsum + k) * W + c];
    if (y2) s += y2[i];
    const float r = x[i] + (tanhf(a1 * s) * w1[c] + b1[c]);
    x[i] = r;
    if (out2) stf(out2, i, tanhf(a2 * r) * w2[c] + b2[c]);
  }
}

// r = y * silu(z) is formed FIRST; then every one of the `ng` equal slices r_k of a row is scaled by
// rsqrt(mean(r_k^2) + eps) and multiplied by w.
template <typename OT>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ldz,
                                           const float* __restrict__ w, OT* __restrict__ out, int inner, int ng, float eps) {
  griddep_launch();
  griddep_wait();
  extern __shared__ float sv[];
  __shared__ float red[32];
  const int t = blockIdx.x, g = blockIdx.y, gs = inner / ng;
  const float* yr = y + (int64_t)t * inner + g * gs;
  const float* zr = z + (int64_t)t * ldz + g * gs;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float v = yr[i] * silu_f(zr[i]);
    sv[i] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float inv = 1.0f / sqrtf(red[0] / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x)
    stf(out, (int64_t)t * inner + g * gs + i, sv[i] * inv * w[g * gs + i]);
}

// gu [T, 2 ff] (gate columns first): out = min(g, limit) * sigmoid(1.702 g') * (clamp(u, -limit, limit) + 1), g' the clamped gate
template <typename OT>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, OT* __restrict__ out, int ff, float limit, int64_t total) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / ff;
    const int c = (int)(i - t * ff);
    const float g = fminf(gu[t * 2 * ff + c], limit);
    const float u = fminf(fmaxf(gu[t * 2 * ff + ff + c], -limit), limit);
    stf(out, i, g / (1.0f + expf(-1.702f * g)) * (u + 1.0f));
  }
}

static inline int flat_grid(int64_t total, int threads) {
  int64_t b = (total + threads - 1) / threads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_embed_scale(const int32_t* tokens, const void* table, int table_dtype, float* out, int T, int W, int V, float scale,
                     void* stream) {
  B200_REQUIRE(tokens && table && out, "embed_scale: null pointer");
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(table_dtype, WT,
                     B200_CUDA_OK(launch_kernel(embed_scale_kernel<WT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, tokens,
                                                (const WT*)table, out, W, V, scale)));
  return B200_OK;
}

int b200_dyt_norm(const float* x, const float* w, const float* b, float alpha, void* out, int out_dtype, int T, int W,
                  void* stream) {
  B200_REQUIRE(x && w && b && out, "dyt_norm: null pointer");
  if (T <= 0) return B200_OK;
  const int64_t total = (int64_t)T * W;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(dyt_kernel<OT>, dim3(flat_grid(total, 256)), dim3(256), 0, (cudaStream_t)stream,
                                                x, w, b, alpha, (OT*)out, W, total)));
  return B200_OK;
}

int b200_dyt_residual(float* x, const float* y, int nsum, const float* y2, const float* w1, const float* b1, float alpha1,
                      const float* w2, const float* b2, float alpha2, void* out2, int out_dtype, int T, int W, void* stream) {
  B200_REQUIRE(x && y && w1 && b1 && nsum >= 1, "dyt_residual: null pointer");
  B200_REQUIRE(!out2 || (w2 && b2), "dyt_residual: the second norm needs its weight and bias");
  if (T <= 0) return B200_OK;
  const int64_t total = (int64_t)T * W;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(dyt_residual_kernel<OT>, dim3(flat_grid(total, 256)), dim3(256), 0,
                                                (cudaStream_t)stream, x, y, nsum, y2, w1, b1, alpha1, w2, b2, alpha2, (OT*)out2,
                                                W, total)));
  return B200_OK;
}

int b200_gated_group_rmsnorm(const float* y, const float* z, int ldz, const float* w, void* out, int out_dtype, int T,
                             int inner, int groups, float eps, void* stream) {
  B200_REQUIRE(y && z && w && out, "gated_group_rmsnorm: null pointer");
  B200_REQUIRE(groups >= 1 && inner % groups == 0, "gated_group_rmsnorm: %d channels do not split into %d groups", inner, groups);
  B200_REQUIRE((size_t)(inner / groups) * 4 <= 160 * 1024, "gated_group_rmsnorm: group of %d too wide", inner / groups);
  if (T <= 0) return B200_OK;
  const size_t smem = (size_t)(inner / groups) * 4;
  B200_DISPATCH_ELEM(out_dtype, OT, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(gated_group_rmsnorm_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_OK(launch_kernel(gated_group_rmsnorm_kernel<OT>, dim3(T, groups), dim3(256), smem, (cudaStream_t)stream, y, z, ldz,
                               w, (OT*)out, inner, groups, eps));
  });
  return B200_OK;
}

int b200_clamped_glu(const float* gate_up, void* out, int out_dtype, int T, int ff, float limit, void* stream) {
  B200_REQUIRE(gate_up && out, "clamped_glu: null pointer");
  if (T <= 0) return B200_OK;
  const int64_t total = (int64_t)T * ff;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(clamped_glu_kernel<OT>, dim3(flat_grid(total, 256)), dim3(256), 0,
                                                (cudaStream_t)stream, gate_up, (OT*)out, ff, limit, total)));
  return B200_OK;
}

}  // extern "C"
