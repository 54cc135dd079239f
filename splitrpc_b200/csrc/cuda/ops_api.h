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
// `bells`: device-visible addresses of 32-bit doorbell words (may be empty).  A launch with bell_value != 0 stores that
// value into every bell once all bytes of the list are in place, then done_value into *done_word (if non-null): the
// gather rings the slot doorbells itself.
uintptr_t srpc_sg_list_create(const std::vector<SgTuple>& items, const std::vector<uint64_t>& bells);
void srpc_sg_list_destroy(uintptr_t handle);
cudaError_t srpc_sg_list_launch(uintptr_t handle, int impl, int n_blocks, cudaStream_t stream, uint32_t bell_value,
                                uintptr_t done_word, uint32_t done_value);
// The same list run through the fused gather + ResNet-stem deserialisation kernel (see sg_kernels.cuh).
cudaError_t srpc_sg_list_launch_stem_s2d(uintptr_t handle, uint64_t ring_base, uint32_t slot_bytes, const float mean[3],
                                         const float inv_std[3], int n_blocks, cudaStream_t stream, uint32_t bell_value,
                                         uintptr_t done_word, uint32_t done_value);
