// Optimizer step of the memory bank from a compact (touched-chapters-only) gradient.
//
// The reference trains the bank with torch.optim.AdamW over all of its rows (training/trainer.py:372-378): rows whose
// chapters no sequence selected have a zero gradient, but their moments still decay, the decoupled weight decay still
// shrinks them and the decayed momentum still moves them.  Parity therefore needs every row visited; what a compact
// gradient saves is the dense gradient tensor itself (805 MB written by torch.gather's backward, read by the
// optimizer, all-reduced by DDP).  One pass, HBM bound: reads and writes the parameter and both moments once
// (6 x 805 MB at the paper shape), reads the compact rows once, and optionally writes the bf16 working copy of the
// bank that the TMA-gather projection reads, so no separate cast pass follows an update.
#include <math.h>

#include "moc_common.cuh"

namespace moc {
namespace {

// slot_of[c] = position of chapter c in the compact list, or -1
__global__ void chapter_slots_kernel(const int* __restrict__ uniq, const int* __restrict__ num_unique,
                                     int max_unique, int C, int* __restrict__ slot_of, int* __restrict__ status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_unique || i >= num_unique[0]) return;
  const int c = uniq[i];
  if (c < 0 || c >= C) { atomicMax(status, MOC_DEV_BAD_INDEX); return; }
  slot_of[c] = i;
}

struct AdamW {
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  float step_size;          // lr / (1 - beta1^t)
  float inv_bc2_sqrt;       // 1 / sqrt(1 - beta2^t)
};

// four consecutive elements per thread; rows are `dim` wide (dim % 4 == 0), chapter = row / T
__global__ void __launch_bounds__(256)
bank_adamw_kernel(float* __restrict__ param, float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
                  const float* __restrict__ grad_rows, const int* __restrict__ slot_of,
                  __nv_bfloat16* __restrict__ shadow, long long total4, int dim4, int T, AdamW h) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / dim4;
    const int c4 = static_cast<int>(i - row * dim4);
    const long long chapter = row / T;
    const int slot = slot_of[chapter];
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    if (slot >= 0) {
      g = reinterpret_cast<const float4*>(grad_rows)[(static_cast<long long>(slot) * T + (row - chapter * T)) * dim4 + c4];
      g.x *= h.grad_scale; g.y *= h.grad_scale; g.z *= h.grad_scale; g.w *= h.grad_scale;
    }
    float4 p = reinterpret_cast<float4*>(param)[i];
    float4 m = reinterpret_cast<float4*>(exp_avg)[i];
    float4 v = reinterpret_cast<float4*>(exp_avg_sq)[i];
    const float decay = 1.f - h.lr * h.weight_decay, w1 = 1.f - h.beta1, w2 = 1.f - h.beta2;
#define MOC_ADAMW_ONE(X)                                                     \
    p.X *= decay;                                                            \
    m.X = m.X + w1 * (g.X - m.X);                       /* lerp */           \
    v.X = v.X * h.beta2 + w2 * g.X * g.X;                                    \
    p.X = p.X - h.step_size * (m.X / (sqrtf(v.X) * h.inv_bc2_sqrt + h.eps));
    MOC_ADAMW_ONE(x) MOC_ADAMW_ONE(y) MOC_ADAMW_ONE(z) MOC_ADAMW_ONE(w)
#undef MOC_ADAMW_ONE
    reinterpret_cast<float4*>(param)[i] = p;
    reinterpret_cast<float4*>(exp_avg)[i] = m;
    reinterpret_cast<float4*>(exp_avg_sq)[i] = v;
    if (shadow != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(p.x, p.y);
      o.y = pack_bf16x2(p.z, p.w);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
}

// partial[block] = sum of squares of the block's share of the compact rows (valid rows only)
__global__ void __launch_bounds__(256)
rows_sqnorm_kernel(const float* __restrict__ rows, const int* __restrict__ num_unique, long long row_elems,
                   float* __restrict__ partial) {
  __shared__ float red[8];
  const long long n = static_cast<long long>(num_unique[0]) * row_elems;
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float x = rows[i];
    acc = fmaf(x, x, acc);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}
__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += 32) acc += partial[i];
  acc = warp_sum(acc);
  if (threadIdx.x == 0) out[0] = acc;
}

constexpr int kNormBlocks = 592;     // 148 SMs x 4

}  // namespace
}  // namespace moc

using namespace moc;

extern "C" size_t moc_bank_adamw_workspace_bytes(int32_t num_chapters) {
  return static_cast<size_t>(num_chapters > 0 ? num_chapters : 0) * sizeof(int32_t);
}

extern "C" int moc_bank_adamw_step(float* param, float* exp_avg, float* exp_avg_sq, int64_t bank_rows, int32_t dim,
                                   int32_t T, const int32_t* uniq, const int32_t* num_unique, int32_t max_unique,
                                   const float* grad_rows, float grad_scale, float lr, float beta1, float beta2,
                                   float eps, float weight_decay, int64_t step, void* shadow_bf16, void* workspace,
                                   size_t workspace_bytes, int32_t* status, void* stream_) {
  MOC_REQUIRE(param && exp_avg && exp_avg_sq && uniq && num_unique && grad_rows && workspace && status, "NULL buffer");
  MOC_REQUIRE(bank_rows > 0 && dim > 0 && T > 0 && bank_rows % T == 0, "bank rows must be whole chapters");
  MOC_REQUIRE(dim % 4 == 0, "row width must be a multiple of 4");
  MOC_REQUIRE(step >= 1, "step counts from 1");
  MOC_REQUIRE(max_unique >= 0, "max_unique must be >= 0");
  for (const void* p : {static_cast<const void*>(param), static_cast<const void*>(exp_avg),
                        static_cast<const void*>(exp_avg_sq), static_cast<const void*>(grad_rows)})
    MOC_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, "buffers must be 16-byte aligned");
  const int C = static_cast<int>(bank_rows / T);
  MOC_REQUIRE(workspace_bytes >= static_cast<size_t>(C) * sizeof(int32_t), "optimizer workspace too small");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int* slot_of = static_cast<int*>(workspace);
  MOC_CUDA_OK(cudaMemsetAsync(slot_of, 0xFF, static_cast<size_t>(C) * sizeof(int32_t), stream));   // all -1
  if (max_unique > 0)
    chapter_slots_kernel<<<ceil_div(max_unique, 256), 256, 0, stream>>>(uniq, num_unique, max_unique, C, slot_of, status);
  AdamW h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = weight_decay; h.grad_scale = grad_scale;
  const double bc1 = 1.0 - pow(static_cast<double>(beta1), static_cast<double>(step));
  const double bc2 = 1.0 - pow(static_cast<double>(beta2), static_cast<double>(step));
  h.step_size = static_cast<float>(static_cast<double>(lr) / bc1);
  h.inv_bc2_sqrt = static_cast<float>(1.0 / sqrt(bc2));
  const long long total4 = bank_rows * (dim / 4);
  long long blocks = (total4 + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  bank_adamw_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(param, exp_avg, exp_avg_sq, grad_rows, slot_of,
                                                                  static_cast<__nv_bfloat16*>(shadow_bf16), total4,
                                                                  dim / 4, T, h);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}

extern "C" int moc_rows_sqnorm(const float* rows, const int32_t* num_unique, int32_t T, int32_t dim, float* out,
                               void* workspace, size_t workspace_bytes, void* stream_) {
  MOC_REQUIRE(rows && num_unique && out && workspace, "NULL buffer");
  MOC_REQUIRE(T > 0 && dim > 0, "empty rows");
  MOC_REQUIRE(workspace_bytes >= kNormBlocks * sizeof(float), "norm workspace too small (592 floats)");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float* partial = static_cast<float*>(workspace);
  rows_sqnorm_kernel<<<kNormBlocks, 256, 0, stream>>>(rows, num_unique, static_cast<long long>(T) * dim, partial);
  sum_partials_kernel<<<1, 32, 0, stream>>>(partial, kNormBlocks, out);
  MOC_CUDA_OK(cudaGetLastError());
  return MOC_OK;
}
