// Table of compiled kernel variants shared between the instantiation units and
// the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"

namespace ayla_b200 {

struct LaunchArgs {
  CUtensorMap tm_a, tm_b, tm_b2, tm_d;
  KernelParams p;
  int grid;
  int cluster_x;  // 0 = the variant's own cluster width (1 or 2)
  int overlap;    // 1 = the launch may start before the previous launch in the stream ends
  cudaStream_t stream;
};

struct KernelEntry {
  int tile_n, cta_group, epilogue, transposed_out, stages, smem_bytes;
  int kb_per_slot;  // k-blocks one ring slot holds
  int activation;  // 1 = the variant whose epilogue applies the launch's activation
  int lean;        // 1 = the variant without the k-split epilogues
  const void* func;
  cudaError_t (*launch)(const LaunchArgs&);
};

constexpr int kMaxSmem = 232448;

template <int BN, int CG, int EPI, bool TR>
constexpr int max_stages() {
  using T1 = GemmTraits<BN, CG, EPI, TR, 1>;
  const int fixed = T1::STORE_BYTES + T1::BIAS_BYTES + T1::MISC_BYTES;
  const int s = (kMaxSmem - fixed) / T1::SLOT_BYTES;
#ifdef AYLA_B200_STAGE_CAP
  return s > AYLA_B200_STAGE_CAP ? AYLA_B200_STAGE_CAP : s;
#else
  return s > 12 ? 12 : s;
#endif
}

template <class T>
cudaError_t launch_variant(const LaunchArgs& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(a.grid), 1, 1);
  cfg.blockDim = dim3(T::THREADS, 1, 1);
  cfg.dynamicSmemBytes = T::SMEM_BYTES;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  const int cluster_x = a.cluster_x > 0 ? a.cluster_x : T::CTA_GROUP;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (a.overlap) {
    // The kernel waits for its predecessor itself (griddepcontrol.wait) before it touches
    // global memory, so its set-up may run under the predecessor's tail.
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, gemm_sm100_kernel<T>, a.tm_a, a.tm_b, a.tm_b2, a.tm_d, a.p);
}

template <int BN, int CG, int EPI, bool TR, bool ACT = false, bool LEAN = false>
KernelEntry make_entry() {
  using T = GemmTraits<BN, CG, EPI, TR, max_stages<BN, CG, EPI, TR>(), ACT, LEAN>;
  KernelEntry e;
  e.tile_n = BN;
  e.cta_group = CG;
  e.epilogue = EPI;
  e.transposed_out = TR ? 1 : 0;
  e.stages = T::STAGES;
  e.smem_bytes = T::SMEM_BYTES;
  e.kb_per_slot = T::KB_PER_SLOT;
  e.activation = ACT ? 1 : 0;
  e.lean = LEAN ? 1 : 0;
  e.func = reinterpret_cast<const void*>(&gemm_sm100_kernel<T>);
  e.launch = &launch_variant<T>;
  return e;
}

// Each instantiation unit contributes its variants.
void append_variants_cg1(KernelEntry* out, int* count);
void append_variants_cg2(KernelEntry* out, int* count);
void append_variants_trans(KernelEntry* out, int* count);
void append_variants_swiglu(KernelEntry* out, int* count);
void append_variants_act_cg1(KernelEntry* out, int* count);
void append_variants_act_cg2(KernelEntry* out, int* count);
void append_variants_act_trans(KernelEntry* out, int* count);
void append_variants_lean_cg1(KernelEntry* out, int* count);
void append_variants_lean_cg2(KernelEntry* out, int* count);
void append_variants_lean_trans(KernelEntry* out, int* count);
void append_variants_lean_act_cg1(KernelEntry* out, int* count);
void append_variants_lean_act_cg2(KernelEntry* out, int* count);
void append_variants_lean_act_trans(KernelEntry* out, int* count);

}  // namespace ayla_b200
