// Gated delta-rule linear attention: causal depthwise conv + SiLU, gates, state recurrence and the gated
// output norm.  Semantics (runtime/nvidia/op_qwen_gdn.cuh:1237-1247, runtime/common/dev_isa.h:1259-1280):
//   x      = SiLU(conv1d_causal(qkv, width W))               per channel, history [W-1] kept per sequence
//   q, k   = x_q / sqrt(|x_q|^2 + 1e-6), x_k / sqrt(|x_k|^2 + 1e-6)       per key head (128 dims)
//   alpha  = exp(-exp(A_log) * softplus(a + dt_bias)),  beta = bf16(sigmoid(b))
//   S     <- alpha S;   S <- S + beta (v - S k) (x) k;   o = S q / sqrt(d)       S[V][K] f32 per (sequence, v head)
//   out    = RMSNorm(o) * gamma * SiLU(z)                                  per (token, v head)
//
// One CTA per (run of consecutive rows of one sequence, v head): 128 threads, thread i owns channel i of
// the head's q / k / v for the conv and row i of S for the recurrence (128 f32 in registers, so the
// per-token update needs no cross-thread traffic beyond the two 128-wide norms and the broadcast of q and
// k through shared memory).  The state is moved between global memory and the registers through a padded
// shared-memory tile so both directions are fully coalesced; a decode step is one 64 KB read + one 64 KB
// write per (sequence, head) and runs at memory speed, a prefill chunk walks its tokens in order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"

namespace {

constexpr int kD = 128;          // head dim = threads per CTA
constexpr int kConvMax = 4;

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ float block_sum128(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  const float s = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  return s;
}

__global__ void __launch_bounds__(kD)
gdn_kernel(__nv_bfloat16* out, float* conv_state, float* ssm_state, const __nv_bfloat16* qkvz, int ld_qkvz,
           const __nv_bfloat16* ba, int ld_ba, const float* conv_w, const float* a_log, const float* dt_bias,
           const int* pos, const int* seq, int rows, int hk, int hv, int conv) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int r0 = blockIdx.x, h = blockIdx.y;
  if (pos[r0] < 0) return;
  if (r0 > 0 && pos[r0 - 1] >= 0 && seq[r0 - 1] == seq[r0] && pos[r0 - 1] + 1 == pos[r0]) return;   // not a run start
  int n = 1;
  while (r0 + n < rows && seq[r0 + n] == seq[r0] && pos[r0 + n] == pos[r0 + n - 1] + 1) ++n;
  extern __shared__ float sm[];
  float* tile = sm;                     // [128][129] state staging
  float* qs = sm + kD * (kD + 1);       // [128]
  float* ks = qs + kD;                  // [128]
  float* red = ks + kD;                 // [4]
  const int i = threadIdx.x;
  const int slot = seq[r0];
  const int rep = hv / hk, kh = h / rep;
  const int C = (2 * hk + hv) * kD;
  const int cq = kh * kD + i, ck = hk * kD + kh * kD + i, cv = 2 * hk * kD + h * kD + i;
  const bool fresh = pos[r0] == 0;
  // ---- state in: coalesced global -> padded smem -> one row per thread
  float S[kD];
  float* Sg = ssm_state + (static_cast<size_t>(slot) * hv + h) * kD * kD;
  if (fresh) {
#pragma unroll
    for (int c = 0; c < kD; ++c) S[c] = 0.f;
  } else {
    for (int e = i; e < kD * kD; e += kD) tile[(e >> 7) * (kD + 1) + (e & 127)] = Sg[e];
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kD; ++c) S[c] = tile[i * (kD + 1) + c];
  }
  // ---- conv taps and history (x[t-3], x[t-2], x[t-1]) of this thread's three channels
  float wq[kConvMax], wk[kConvMax], wv[kConvMax], hq[kConvMax - 1], hkk[kConvMax - 1], hvv[kConvMax - 1];
  constexpr int W = kConvMax;   // the launcher admits width 4 only
  (void)conv;
#pragma unroll
  for (int j = 0; j < kConvMax; ++j) {
    wq[j] = j < W ? conv_w[cq * W + j] : 0.f;
    wk[j] = j < W ? conv_w[ck * W + j] : 0.f;
    wv[j] = j < W ? conv_w[cv * W + j] : 0.f;
  }
  float* cs = conv_state + static_cast<size_t>(slot) * C * (W - 1);
#pragma unroll
  for (int j = 0; j < kConvMax - 1; ++j) {
    const bool have = !fresh && j < W - 1;
    hq[j] = have ? cs[cq * (W - 1) + j] : 0.f;
    hkk[j] = have ? cs[ck * (W - 1) + j] : 0.f;
    hvv[j] = have ? cs[cv * (W - 1) + j] : 0.f;
  }
  const float neg_ea = -__expf(a_log[h]), dtb = dt_bias[h];
  const float scale = rsqrtf(static_cast<float>(kD));
  for (int t = 0; t < n; ++t) {
    const int r = r0 + t;
    const __nv_bfloat16* x = qkvz + static_cast<size_t>(r) * ld_qkvz;
    const float xq = __bfloat162float(x[cq]), xk = __bfloat162float(x[ck]), xv = __bfloat162float(x[cv]);
    // taps are ordered oldest first: history holds the W-1 previous inputs, the newest tap is this token
    float aq = wq[W - 1] * xq, ak = wk[W - 1] * xk, av = wv[W - 1] * xv;
#pragma unroll
    for (int j = 0; j < kConvMax - 1; ++j) {
      if (j < W - 1) { aq = fmaf(wq[j], hq[j], aq); ak = fmaf(wk[j], hkk[j], ak); av = fmaf(wv[j], hvv[j], av); }
    }
#pragma unroll
    for (int j = 0; j < kConvMax - 2; ++j) {
      if (j < W - 2) { hq[j] = hq[j + 1]; hkk[j] = hkk[j + 1]; hvv[j] = hvv[j + 1]; }
    }
    if (W >= 2) { hq[W - 2] = xq; hkk[W - 2] = xk; hvv[W - 2] = xv; }
    const float q = silu(aq), k = silu(ak), v = silu(av);
    const float qn = block_sum128(q * q, red), kn = block_sum128(k * k, red);
    qs[i] = q * rsqrtf(qn + 1e-6f);
    ks[i] = k * rsqrtf(kn + 1e-6f);
    const float bb = __bfloat162float(ba[static_cast<size_t>(r) * ld_ba + h]);
    const float aa = __bfloat162float(ba[static_cast<size_t>(r) * ld_ba + hv + h]) + dtb;
    const float sp = aa > 20.f ? aa : log1pf(__expf(aa));
    const float alpha = __expf(neg_ea * sp);
    const float beta = __bfloat162float(__float2bfloat16(1.0f / (1.0f + __expf(-bb))));
    __syncthreads();
    float pred = 0.f;
#pragma unroll
    for (int c = 0; c < kD; ++c) { S[c] *= alpha; pred = fmaf(S[c], ks[c], pred); }
    const float dv = beta * (v - pred);
    float o = 0.f;
#pragma unroll
    for (int c = 0; c < kD; ++c) { S[c] = fmaf(dv, ks[c], S[c]); o = fmaf(S[c], qs[c], o); }
    out[static_cast<size_t>(r) * hv * kD + h * kD + i] = __float2bfloat16(o * scale);
    __syncthreads();   // qs / ks are rewritten by the next token
  }
  // ---- state out
#pragma unroll
  for (int c = 0; c < kD; ++c) tile[i * (kD + 1) + c] = S[c];
  __syncthreads();
  for (int e = i; e < kD * kD; e += kD) Sg[e] = tile[(e >> 7) * (kD + 1) + (e & 127)];
}

// Conv history update, one thread per (run start, channel): new history = the last W-1 inputs of (old history ++ run).
// It runs after gdn_kernel because several v heads of that kernel read the q / k channels of the key head they share;
// updating them from inside it would race with a CTA that has not read the old history yet.
__global__ void gdn_conv_state_kernel(float* conv_state, const __nv_bfloat16* qkvz, int ld_qkvz, const int* pos, const int* seq,
                                      int rows, int C) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  constexpr int W = kConvMax;
  const int r0 = blockIdx.x;
  if (pos[r0] < 0) return;
  if (r0 > 0 && pos[r0 - 1] >= 0 && seq[r0 - 1] == seq[r0] && pos[r0 - 1] + 1 == pos[r0]) return;
  int n = 1;
  while (r0 + n < rows && seq[r0 + n] == seq[r0] && pos[r0 + n] == pos[r0 + n - 1] + 1) ++n;
  const bool fresh = pos[r0] == 0;
  float* cs = conv_state + static_cast<size_t>(seq[r0]) * C * (W - 1);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float h[W - 1];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      const int back = (W - 1) - j;            // this slot holds the input `back` steps before the next token
      h[j] = back <= n ? __bfloat162float(qkvz[static_cast<size_t>(r0 + n - back) * ld_qkvz + c])
                       : (fresh ? 0.f : cs[c * (W - 1) + j + n]);
    }
#pragma unroll
    for (int j = 0; j < W - 1; ++j) cs[c * (W - 1) + j] = h[j];
  }
}

// One warp per (row, head): out = RMSNorm(o) * gamma * SiLU(z).
__global__ void gated_norm_kernel(__nv_bfloat16* out, const __nv_bfloat16* o, const __nv_bfloat16* z, int ld_z, int z_ofs,
                                  const float* gamma, int rows, int heads, int hd, float eps) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wib;
  if (item >= static_cast<long long>(rows) * heads) return;
  const int r = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const __nv_bfloat16* src = o + (static_cast<size_t>(r) * heads + h) * hd;
  float ss = 0.f;
  for (int c = lane; c < hd; c += 32) { const float v = __bfloat162float(src[c]); ss += v * v; }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float rs = rsqrtf(ss / hd + eps);
  for (int c = lane; c < hd; c += 32) {
    const float zz = __bfloat162float(z[static_cast<size_t>(r) * ld_z + z_ofs + h * hd + c]);
    out[(static_cast<size_t>(r) * heads + h) * hd + c] = __float2bfloat16(__bfloat162float(src[c]) * rs * gamma[c] * silu(zz));
  }
}

// out = a * sigmoid(gate)   (gated full-attention layers of the hybrid model)
__global__ void sigmoid_gate_kernel(__nv_bfloat16* out, const __nv_bfloat16* a, const __nv_bfloat16* gate, long long n) {
  plow::pdl_launch_dependents();
  plow::pdl_wait();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(__bfloat162float(a[i]) / (1.0f + __expf(-__bfloat162float(gate[i]))));
}

}  // namespace

extern "C" {

// qkvz bf16 [rows][ld_qkvz] = [q (hk*128) | k (hk*128) | v (hv*128) | z ...]; ba bf16 [rows][ld_ba] = [b (hv) | a (hv)];
// conv_w f32 [(2hk+hv)*128][conv]; conv_state f32 [slots][(2hk+hv)*128][conv-1]; ssm_state f32 [slots][hv][128][128];
// out bf16 [rows][hv*128].  A row whose position is 0 starts its sequence from a zero state.
int plow_gdn(void* out, float* conv_state, float* ssm_state, const void* qkvz, int ld_qkvz, const void* ba, int ld_ba,
             const float* conv_w, const float* a_log, const float* dt_bias, const int* pos, const int* seq, int rows,
             int hk, int hv, int head_dim, int conv, void* stream) {
  if (rows <= 0 || head_dim != kD || conv != kConvMax || hk <= 0 || hv % hk) return -1;
  constexpr int kSmem = (kD * (kD + 1) + 2 * kD + 8) * sizeof(float);
  static plow::DeviceOnce attr;
  if (plow::ensure_smem(attr, gdn_kernel, kSmem) != cudaSuccess) return 3000;
  plow::launch_serial(gdn_kernel, dim3(rows, hv), dim3(kD), kSmem, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16*>(out), conv_state, ssm_state, static_cast<const __nv_bfloat16*>(qkvz), ld_qkvz,
      static_cast<const __nv_bfloat16*>(ba), ld_ba, conv_w, a_log, dt_bias, pos, seq, rows, hk, hv, conv);
  plow::launch_serial(gdn_conv_state_kernel, dim3(rows), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      conv_state, static_cast<const __nv_bfloat16*>(qkvz), ld_qkvz, pos, seq, rows, (2 * hk + hv) * kD);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

int plow_gated_norm(void* out, const void* o, const void* z, int ld_z, int z_ofs, const float* gamma, int rows, int heads,
                    int hd, float eps, void* stream) {
  if (rows <= 0) return -1;
  const long long items = static_cast<long long>(rows) * heads;
  plow::launch_serial(gated_norm_kernel, dim3(static_cast<unsigned>((items + 7) / 8)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(z), ld_z, z_ofs,
      gamma, rows, heads, hd, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

int plow_sigmoid_gate(void* out, const void* a, const void* gate, int64_t n, void* stream) {
  if (n <= 0) return -1;
  plow::launch_serial(sigmoid_gate_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(gate), n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 4000 + static_cast<int>(e);
}

}  // extern "C"
