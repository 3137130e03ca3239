// Stand-in for cutlass/examples/common/helper.h (not shipped with the header-only CUTLASS tree used here):
// the one macro the reference's batch_gemm_softmax.cu takes from it.
#pragma once
#include <stdexcept>
#include <string>
#include "cutlass/cutlass.h"
#define CUTLASS_CHECK(status)                                                                        \
  {                                                                                                  \
    cutlass::Status error = status;                                                                  \
    if (error != cutlass::Status::kSuccess)                                                          \
      throw std::runtime_error(std::string("CUTLASS error: ") + cutlassGetStatusString(error));      \
  }
