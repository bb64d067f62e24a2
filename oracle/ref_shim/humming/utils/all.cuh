// Host-compilation shim, found before the reference's own humming/utils/all.cuh
// on the include path.  The reference's all.cuh pulls in inline-PTX helpers
// that only nvcc device passes accept; the two headers compiled for the oracle
// check (kernel/pack_weight.cuh, kernel/dequant_weight.cuh) need nothing from
// it beyond the macros of utils/base.cuh.
#pragma once
#include <humming/utils/base.cuh>
