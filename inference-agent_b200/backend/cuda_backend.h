// CUDA (B200, sm_100a) backend for Ingot: implements the Backend interface of src/backend.h with the
// attention stage running through libingot_cuda.so (include/ingot_cuda.h).
#pragma once

#include <memory>

#include "backend.h"
#include "gguf.h"
#include "model.h"

// Same contract as make_metal_backend (src/metal_backend.h:13): throws std::runtime_error if no CUDA
// device is usable or the model holds a tensor type this backend does not read.
// n_batch is the most tokens one forward_batch call may process at once.
std::unique_ptr<Backend> make_cuda_backend(const gguf::File& file, const Model& model, int n_ctx, int n_batch);
