// Tensor-parallel communicator: one NCCL communicator per process (one process per GPU), loaded at
// run time so the library has no link-time NCCL dependency and shares the copy the launcher's
// framework may already have loaded.
#pragma once

#include <cstdint>

namespace bfb200 {

void tpUniqueId(void* hostId128);
void tpInit(const void* hostId128, int rank, int world);
// In-place sum over all ranks on `stream`; dtype is BFB_F32 or BFB_BF16.
void tpAllReduceSum(void* deviceBuffer, std::int64_t count, int dtype, void* stream);
// In-place average over all ranks of `tensors` fp32 gradient buffers, issued as one group on `stream`: replaces the
// reference's host-staged average (download every replica's gradient, add and scale on the host, upload to every
// replica; src/backend/cuda/multi_gpu_train_runner.cu:275-297).
void tpAverageGradients(void* const* deviceBuffers, const std::int64_t* counts, int tensors, void* stream);
void tpDestroy();
bool tpReady();
// Waits for `stream` like cudaStreamSynchronize, but with a deadline (BFB_TP_TIMEOUT_MS, default 120 s) while a
// communicator exists: polls the stream and the communicator's asynchronous error state and aborts the communicator
// when the deadline passes or it reports an error (BFB_TIMEOUT / BFB_CUDA_ERROR), so that a rank that is missing
// from a collective cannot block the others for ever. Without a communicator it is a plain synchronize.
void tpSynchronize(void* stream);

}  // namespace bfb200
