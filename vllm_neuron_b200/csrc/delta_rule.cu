// Gated delta-rule recurrence over a ragged batch, beside the selective state-space scan (ssm_scan.cu).
// Per head, token by token, with a matrix state S [D keys x P values] in fp32:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (o sees the token's own write)
//   * delta_prep: per token, q and k (after their short convolution) become unit vectors per key head,
//     x / sqrt(sum x^2 + unit_eps), q also times q_scale; beta = sigmoid(raw_b), g = exp(-exp(A_log) softplus(raw_a + dt_bias));
//     k . q per key head is kept for the read-out.  Everything fp32.
//   * delta_scan: the columns of S evolve independently (column j only needs v_j), so a CTA owns PC columns of one head of
//     one sequence and L lanes share a column, each keeping R rows in registers: groups of four consecutive rows dealt
//     round-robin to the lanes (lane l holds rows 4 L i + 4 l .. + 3, i < R / 4), so that the lanes of a column read
//     consecutive 16-byte pieces of the staged k and q rows (no bank conflicts) and of the state.  With s_k = S^T k and
//     s_q = S^T q taken BEFORE the update (one pass over the registers, one shuffle tree for both),
//         u = beta (v - g s_k),   S <- g S + k u,   o = g s_q + u (k . q)
//     is the recurrence above, term for term; the kernel takes the tokens two at a time (see the loop), which halves
//     the number of dependent reductions.  Tokens are staged through shared memory in chunks, a ring of DS_STAGES
//     buffers whose cp.async copies run three chunks ahead of the steps (a chunk's steps take about as long as one trip to
//     HBM, so one chunk of lead does not hide it).  State layout [slots][H][P][D] (a column's rows are
//     contiguous), read when the sequence continues (pos0 > 0), zero otherwise, written back at the end of the portion.
#include <math.h>

#include "hybrid_common.cuh"

namespace b200 {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// one CTA per token: warps take the key heads (unit norms, k . q), threads the value heads (beta, decay)
__global__ void delta_prep_kernel(float* __restrict__ qkv, int ldc, const float* __restrict__ proj, int ldp, int b_col0, int a_col0,
                                  const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ bg,
                                  float* __restrict__ kq, int H, int G, int D, float q_scale, float unit_eps) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < G; g += nw) {
    float* q = qkv + (int64_t)t * ldc + (int64_t)g * D;
    float* k = q + (int64_t)G * D;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < D; i += 32) {
      sq += q[i] * q[i];
      sk += k[i] * k[i];
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float iq = q_scale / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
    float dot = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float a = q[i] * iq, b = k[i] * ik;
      q[i] = a;
      k[i] = b;
      dot += a * b;
    }
    dot = warp_sum(dot);
    if (lane == 0) kq[(int64_t)t * G + g] = dot;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float rb = proj[(int64_t)t * ldp + b_col0 + h], ra = proj[(int64_t)t * ldp + a_col0 + h];
    bg[(int64_t)t * 2 * H + h] = 1.0f / (1.0f + expf(-rb));
    bg[(int64_t)t * 2 * H + H + h] = expf(-expf(A_log[h]) * softplus_f(ra + dt_bias[h]));
  }
}

constexpr int DS_THREADS = 128;
constexpr int DS_STAGES = 4;
constexpr int DS_CHUNK = 16;  // tokens staged per shared-memory buffer (fewer when the key rows are long: the two stages must fit)

template <int N>
__device__ __forceinline__ void cp_async_f32(uint32_t dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(dst), "l"(src), "n"(N * 4) : "memory");
}

// grid (P / PC column chunks, H, sequences); thread = (column cl = tid / L, lane part l = tid % L), rows 4 L i + 4 l + {0..3}
template <int R>
__global__ void __launch_bounds__(DS_THREADS)
    delta_scan_kernel(const float* __restrict__ qkv, int ldc, const float* __restrict__ bg, const float* __restrict__ kq,
                      float* __restrict__ state, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                      const int32_t* __restrict__ seq_pos0, float* __restrict__ out, int H, int G, int D, int P, int L, int vec4, int CH) {
  griddep_wait();
  const int sq = blockIdx.z, h = blockIdx.y, PC = DS_THREADS / L, c0 = blockIdx.x * PC;
  const int t0 = seq_start[sq], n = seq_start[sq + 1] - t0;
  if (n <= 0) return;
  const int g = h / (H / G);
  const int Dp = L * R;  // padded key length: rows past D stay zero
  extern __shared__ __align__(16) float ds_sm[];
  // per stage: q [CH][Dp] | k [CH][Dp] | v [CH][PC] | beta, decay, k.q [3][CH]
  const int stage_f = CH * (2 * Dp + PC + 3);
  float* o_s = ds_sm + DS_STAGES * stage_f;  // [CH][PC]
  const int tid = threadIdx.x, cl = tid / L, l = tid - cl * L;
  const int col = c0 + cl;
  const bool col_ok = col < P;
  for (int i = tid; i < DS_STAGES * stage_f; i += DS_THREADS) ds_sm[i] = 0.f;  // the pads (rows past D, columns past P) stay zero
  __syncthreads();
  const uint32_t sm0 = smem_u32(ds_sm);
  const int vcols = P - c0 < PC ? P - c0 : PC;
  // this thread's first copy of a chunk and the step to its next one (rows of dq / vq 16-byte pieces, or D / vcols floats):
  // the divisions happen once, not per chunk
  const int dq = vec4 ? D >> 2 : D, vq = vec4 ? vcols >> 2 : vcols;
  const int q_r0 = tid / dq, q_d0 = tid - q_r0 * dq, q_dr = DS_THREADS / dq, q_dd = DS_THREADS - q_dr * dq;
  const int v_r0 = vq > 0 ? tid / vq : CH, v_d0 = vq > 0 ? tid - v_r0 * vq : 0, v_dr = vq > 0 ? DS_THREADS / vq : 0,
            v_dd = vq > 0 ? DS_THREADS - v_dr * vq : 0;
  const float* src_q0 = qkv + (int64_t)t0 * ldc + (int64_t)g * D;
  const float* src_v0 = qkv + (int64_t)t0 * ldc + 2 * (int64_t)G * D + (int64_t)h * P + c0;
  const int64_t k_off = (int64_t)G * D;
  auto issue = [&](int ck) {
    const int i0 = ck * CH;
    const int cnt = n - i0 < CH ? n - i0 : CH;
    if (cnt > 0) {
      const uint32_t base = sm0 + (uint32_t)((ck % DS_STAGES) * stage_f * 4);
      const float* src_q = src_q0 + (int64_t)i0 * ldc;
      const float* src_v = src_v0 + (int64_t)i0 * ldc;
      for (int r = q_r0, d = q_d0; r < cnt;) {
        if (vec4) {
          cp_async_f32<4>(base + (uint32_t)((r * Dp + 4 * d) * 4), src_q + (int64_t)r * ldc + 4 * d);
          cp_async_f32<4>(base + (uint32_t)(((CH + r) * Dp + 4 * d) * 4), src_q + k_off + (int64_t)r * ldc + 4 * d);
        } else {
          cp_async_f32<1>(base + (uint32_t)((r * Dp + d) * 4), src_q + (int64_t)r * ldc + d);
          cp_async_f32<1>(base + (uint32_t)(((CH + r) * Dp + d) * 4), src_q + k_off + (int64_t)r * ldc + d);
        }
        r += q_dr;
        d += q_dd;
        if (d >= dq) {
          d -= dq;
          ++r;
        }
      }
      for (int r = v_r0, d = v_d0; r < cnt;) {
        if (vec4) cp_async_f32<4>(base + (uint32_t)((2 * CH * Dp + r * PC + 4 * d) * 4), src_v + (int64_t)r * ldc + 4 * d);
        else cp_async_f32<1>(base + (uint32_t)((2 * CH * Dp + r * PC + d) * 4), src_v + (int64_t)r * ldc + d);
        r += v_dr;
        d += v_dd;
        if (d >= vq) {
          d -= vq;
          ++r;
        }
      }
      const uint32_t sc = base + (uint32_t)((CH * (2 * Dp + PC)) * 4);
      for (int i = tid; i < cnt; i += DS_THREADS) {
        cp_async_f32<1>(sc + (uint32_t)(i * 4), bg + (int64_t)(t0 + i0 + i) * 2 * H + h);
        cp_async_f32<1>(sc + (uint32_t)((CH + i) * 4), bg + (int64_t)(t0 + i0 + i) * 2 * H + H + h);
        cp_async_f32<1>(sc + (uint32_t)((2 * CH + i) * 4), kq + (int64_t)(t0 + i0 + i) * G + g);
      }
    }
    cp_async_commit();  // an empty group past the end keeps the wait counts uniform
  };
  // ---- state
  float S[R];
  float* srow = state + (((int64_t)seq_slot[sq] * H + h) * P + (col_ok ? col : 0)) * D + 4 * l;
  const int gstep = 4 * L;  // rows between two of this lane's groups of four
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = 0.f;
  if (seq_pos0[sq] > 0 && col_ok) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if ((r >> 2) * gstep + 4 * l + (r & 3) < D) S[r] = srow[(r >> 2) * gstep + (r & 3)];
  }
  const int chunks = (n + CH - 1) / CH;
#pragma unroll
  for (int i = 0; i < DS_STAGES - 1; ++i) issue(i);
  for (int ck = 0; ck < chunks; ++ck) {
    issue(ck + DS_STAGES - 1);  // into the stage chunk ck - 1 used: everyone left it at the barrier that ended that chunk
    cp_async_wait<DS_STAGES - 1>();
    __syncthreads();  // chunk ck of every thread has landed; o_s of chunk ck - 1 has been flushed
    const float* st = ds_sm + (ck % DS_STAGES) * stage_f;
    const float* qs = st + 4 * l;
    const float* ks = st + CH * Dp + 4 * l;
    const float* vs = st + 2 * CH * Dp + cl;
    const float* sc = st + CH * (2 * Dp + PC);
    const int cnt = n - ck * CH < CH ? n - ck * CH : CH;
    int c = 0;
    // ---- two tokens per round: with a = S^T k1, b = S^T k2, cq = S^T q1, d = S^T q2 and the scalars e = k1 . k2,
    // f = k1 . q2 (all six reduced over the lanes in ONE shuffle tree),
    //     u1 = beta1 (v1 - g1 a)                 o1 = g1 cq + u1 (k1 . q1)
    //     u2 = beta2 (v2 - g2 (g1 b + e u1))     o2 = g2 (g1 d + f u1) + u2 (k2 . q2)
    //     S <- g1 g2 S + (g2 u1) k1 + u2 k2
    // which is two steps of the recurrence with half the dependent reductions.
    for (; c + 1 < cnt; c += 2) {
      // packed fp32 pairs: rows (r, r + 1) of the state, k and q go through one fma.rn.f32x2 each
      float2 k1[R / 2], k2[R / 2];
      float2 a2 = make_float2(0.f, 0.f), b2 = a2, c2 = a2, d2 = a2, e2 = a2, f2 = a2;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const int off = c * Dp + (r >> 2) * gstep;
        const float4 ka = *reinterpret_cast<const float4*>(ks + off);
        const float4 qa = *reinterpret_cast<const float4*>(qs + off);
        const float4 kb = *reinterpret_cast<const float4*>(ks + off + Dp);
        const float4 qb = *reinterpret_cast<const float4*>(qs + off + Dp);
        const float2 s0 = make_float2(S[r], S[r + 1]), s1 = make_float2(S[r + 2], S[r + 3]);
        const float2 ka0 = make_float2(ka.x, ka.y), ka1 = make_float2(ka.z, ka.w);
        const float2 kb0 = make_float2(kb.x, kb.y), kb1 = make_float2(kb.z, kb.w);
        const float2 qb0 = make_float2(qb.x, qb.y), qb1 = make_float2(qb.z, qb.w);
        k1[r >> 1] = ka0, k1[(r >> 1) + 1] = ka1;
        k2[r >> 1] = kb0, k2[(r >> 1) + 1] = kb1;
        a2 = ffma2(s1, ka1, ffma2(s0, ka0, a2));
        b2 = ffma2(s1, kb1, ffma2(s0, kb0, b2));
        c2 = ffma2(s1, make_float2(qa.z, qa.w), ffma2(s0, make_float2(qa.x, qa.y), c2));
        d2 = ffma2(s1, qb1, ffma2(s0, qb0, d2));
        e2 = ffma2(ka1, kb1, ffma2(ka0, kb0, e2));
        f2 = ffma2(ka1, qb1, ffma2(ka0, qb0, f2));
      }
      float e0 = e2.x + e2.y, f0 = f2.x + f2.y;
      const float a0 = a2.x, a1 = a2.y, b0 = b2.x, b1 = b2.y, cq0 = c2.x, cq1 = c2.y, d0 = d2.x, d1 = d2.y;
      float a = a0 + a1, b = b0 + b1, cq = cq0 + cq1, d = d0 + d1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        if (o < L) {
          a += __shfl_xor_sync(0xffffffffu, a, o);
          b += __shfl_xor_sync(0xffffffffu, b, o);
          cq += __shfl_xor_sync(0xffffffffu, cq, o);
          d += __shfl_xor_sync(0xffffffffu, d, o);
          e0 += __shfl_xor_sync(0xffffffffu, e0, o);
          f0 += __shfl_xor_sync(0xffffffffu, f0, o);
        }
      }
      const float beta1 = sc[c], g1 = sc[CH + c], kq1 = sc[2 * CH + c];
      const float beta2 = sc[c + 1], g2 = sc[CH + c + 1], kq2 = sc[2 * CH + c + 1];
      const float u1 = beta1 * (vs[c * PC] - g1 * a);
      const float u2 = beta2 * (vs[(c + 1) * PC] - g2 * (g1 * b + e0 * u1));
      const float gg = g1 * g2, w1 = g2 * u1;
      const float2 gg2 = make_float2(gg, gg), w12 = make_float2(w1, w1), u22 = make_float2(u2, u2);
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        const float2 sn = ffma2(k2[r >> 1], u22, ffma2(k1[r >> 1], w12, fmul2(gg2, make_float2(S[r], S[r + 1]))));
        S[r] = sn.x;
        S[r + 1] = sn.y;
      }
      if (l == 0) {
        o_s[c * PC + cl] = g1 * cq + u1 * kq1;
        o_s[(c + 1) * PC + cl] = g2 * (g1 * d + f0 * u1) + u2 * kq2;
      }
    }
    if (c < cnt) {  // an odd token left
      float kr[R];
      float pk0 = 0.f, pk1 = 0.f, pq0 = 0.f, pq1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + c * Dp + (r >> 2) * gstep);
        const float4 q4 = *reinterpret_cast<const float4*>(qs + c * Dp + (r >> 2) * gstep);
        kr[r] = k4.x, kr[r + 1] = k4.y, kr[r + 2] = k4.z, kr[r + 3] = k4.w;
        pk0 += S[r] * k4.x + S[r + 2] * k4.z;
        pk1 += S[r + 1] * k4.y + S[r + 3] * k4.w;
        pq0 += S[r] * q4.x + S[r + 2] * q4.z;
        pq1 += S[r + 1] * q4.y + S[r + 3] * q4.w;
      }
      float pk = pk0 + pk1, pq = pq0 + pq1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        if (o < L) {  // L is a power of two, the same for every thread
          pk += __shfl_xor_sync(0xffffffffu, pk, o);
          pq += __shfl_xor_sync(0xffffffffu, pq, o);
        }
      }
      const float beta = sc[c], gd = sc[CH + c], dkq = sc[2 * CH + c];
      const float u = beta * (vs[c * PC] - gd * pk);
#pragma unroll
      for (int r = 0; r < R; ++r) S[r] = gd * S[r] + kr[r] * u;
      if (l == 0) o_s[c * PC + cl] = gd * pq + u * dkq;
    }
    __syncthreads();  // o_s complete; everyone is done with this stage before the next iteration copies a later chunk into it
    for (int i = tid; i < cnt * vcols; i += DS_THREADS) {
      const int r = i / vcols, d = i - r * vcols;
      out[((int64_t)(t0 + ck * CH + r) * H + h) * P + c0 + d] = o_s[r * PC + d];
    }
  }
  // the next kernel of the stream may take SM slots from here on: earlier, its waiting CTAs would displace this kernel's own
  griddep_launch();
  cp_async_wait<0>();
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if ((r >> 2) * gstep + 4 * l + (r & 3) < D) srow[(r >> 2) * gstep + (r & 3)] = S[r];
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_delta_prep(float* qkv, int ldc, const float* proj, int ldp, int b_col0, int a_col0, const float* A_log,
                    const float* dt_bias, float* beta_decay, float* kq, int T, int H, int G, int D, float q_scale, float unit_eps,
                    void* stream) {
  B200_REQUIRE(qkv && proj && A_log && dt_bias && beta_decay && kq, "delta_prep: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0, "delta_prep: %d heads over %d key heads of %d", H, G, D);
  if (T <= 0) return B200_OK;
  B200_CUDA_OK(launch_kernel(delta_prep_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, qkv, ldc, proj, ldp, b_col0, a_col0,
                             A_log, dt_bias, beta_decay, kq, H, G, D, q_scale, unit_eps));
  return B200_OK;
}

int b200_delta_scan(const float* qkv, int ldc, const float* beta_decay, const float* kq, float* state, const int32_t* seq_start,
                    const int32_t* seq_slot, const int32_t* seq_pos0, float* out, int B, int max_new, int H, int G, int D, int P,
                    void* stream) {
  B200_REQUIRE(qkv && beta_decay && kq && state && seq_start && seq_slot && seq_pos0 && out, "delta_scan: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0, "delta_scan: %d heads over %d key heads", H, G);
  B200_REQUIRE(D >= 1 && D <= 1024 && P >= 1, "delta_scan: key size %d (1..1024 supported)", D);
  if (B <= 0) return B200_OK;
  // L lanes per column (a power of two), R rows per lane.  More rows per lane mean fewer shuffles and shared-memory reads
  // per multiply-add but fewer warps to hide their latency.  Measured at D = 128, 16 heads: one 4096-token portion 1.38 /
  // 0.97 / 1.27 ms at 32 / 16 / 8 rows per lane; 64 single tokens 0.057 / 0.057 / 0.099 ms (they mostly move the state).
  const int rows_target = max_new > 4 ? 16 : 32;
  int L = 1;
  while (L < 32 && L * rows_target < D) L <<= 1;
  const int need = (D + L - 1) / L;
  const int R = need <= 8 ? 8 : need <= 16 ? 16 : 32;
  const int PC = DS_THREADS / L;
  const int vcols_min = P % PC ? P % PC : PC;
  const int vec4 = D % 4 == 0 && ldc % 4 == 0 && P % 4 == 0 && PC % 4 == 0 && vcols_min % 4 == 0 && !((uintptr_t)qkv & 15);
  int CH = DS_CHUNK;
  while (CH > 4 && (size_t)(DS_STAGES * CH * (2 * L * R + PC + 3) + CH * PC) * 4 > 160 * 1024) CH >>= 1;
  const size_t smem = (size_t)(DS_STAGES * CH * (2 * L * R + PC + 3) + CH * PC) * 4;
  dim3 grid((P + PC - 1) / PC, H, B);
  cudaStream_t st = (cudaStream_t)stream;
#define DS_LAUNCH(RR)                                                                                                        \
  do {                                                                                                                       \
    if (smem > 48 * 1024)                                                                                                    \
      B200_CUDA_OK(cudaFuncSetAttribute(delta_scan_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    B200_CUDA_OK(launch_kernel_serial(delta_scan_kernel<RR>, grid, dim3(DS_THREADS), smem, st, qkv, ldc, beta_decay, kq,    \
                                      state, seq_start, seq_slot, seq_pos0, out, H, G, D, P, L, vec4, CH));                 \
  } while (0)
  if (R == 8) DS_LAUNCH(8);
  else if (R == 16) DS_LAUNCH(16);
  else DS_LAUNCH(32);
#undef DS_LAUNCH
  return B200_OK;
}

}  // extern "C"
