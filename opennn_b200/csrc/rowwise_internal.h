// Internal interface between the loss front end (softmax_loss_adam.cu) and the shared-memory staged
// CrossEntropyError3d kernel (ce3d_staged.cu).
#pragma once
#include <cuda_runtime.h>
#include "../../include/onn_b200.h"

namespace onn
{
// Takes rows of at least 4096 and at most 35712 logits, a multiple of 4, 16-byte aligned, no separate probabilities output.
bool ce3d_staged_takes(const float* logits, const float* probabilities_out, long long rows, long long V);
// In place: logits (or probabilities) -> (p - onehot) / active; row_scratch as the two-sweep kernel leaves it.
int ce3d_staged_launch(float* logits, const float* targets, const float* active_count, float* row_scratch,
                       long long rows, int V, int inputs_are_probabilities, cudaStream_t stream);
int ce3d_staged_read_status();
const unsigned int* ce3d_staged_status_word();       // device address on the current device
}
