// Bindings for the ops added after the core training path (elementwise family, quantised
// GEMV, collectives).  Kept separate so touching one group does not recompile the other.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"
#include "common/launch.h"

void register_extra_ops(pybind11::module_& m) { (void)m; }
