// Stand-in for <cooperative_groups.h> when the kernels are compiled for the host emulation (tests only).
#pragma once
#include "../cuda_emu.h"
