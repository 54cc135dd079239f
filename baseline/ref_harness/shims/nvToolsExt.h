// The original includes the NVTX v2 header by this name; CUDA 12.9 ships NVTX v3 only.
#pragma once
#include <nvtx3/nvToolsExt.h>
