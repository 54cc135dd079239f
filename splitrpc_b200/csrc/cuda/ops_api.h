// C++ entry points of the CUDA kernels used by the Python bindings.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <tuple>
#include <vector>

extern "C" int srpc_device_caps(int dev, int* vmm, int* stream_memops, int* gdr_with_vmm, int* sm_major, int* sm_minor,
                                int* n_sm);

using SgTuple = std::tuple<uintptr_t, uintptr_t, uint32_t>;
// One-shot: uploads the list, launches, and returns after the copy finished.
cudaError_t srpc_sg_copy_list(const std::vector<SgTuple>& items, int impl, int n_blocks, cudaStream_t stream);
cudaError_t srpc_sg_cast_list(const std::vector<SgTuple>& items, float scale, float shift, int n_blocks, cudaStream_t stream);
// Resident copy list in device memory for repeated launches (benchmarks, graphs).
uintptr_t srpc_sg_list_create(const std::vector<SgTuple>& items);
void srpc_sg_list_destroy(uintptr_t handle);
cudaError_t srpc_sg_list_launch(uintptr_t handle, int impl, int n_blocks, cudaStream_t stream);
// The same list run through the fused gather + ResNet-stem deserialisation kernel (see sg_kernels.cuh).
cudaError_t srpc_sg_list_launch_stem_s2d(uintptr_t handle, uint64_t ring_base, uint32_t slot_bytes, const float mean[3],
                                         const float inv_std[3], int n_blocks, cudaStream_t stream);
