// Stand-in for <cuda_bf16.h> when the kernels are compiled for the host emulation (tests only).
#pragma once
#include "../cuda_emu.h"
