"""B200 device backend for the pjrt-ocl VMProgram v3 bytecode.

`runtime` mirrors the reference's C++ runtime interface over the C ABI of
`libb2vm.so` (include/b2vm.h); `build` compiles that library for sm_100a.
"""
from .runtime import (B2Error, DeadlineExceeded, FailedPrecondition, Internal,  # noqa: F401
                      InvalidArgument, LoadedProgram, ResourceExhausted, Runtime,
                      Unimplemented, VmProgram, EXPORTS, find_library, lib)

# Tile geometry the device executes with; a lowering subprocess must be given
# exactly these (PJRT_OCL_EW_TS / PJRT_OCL_MMA_T, plugin.cc:770-773).
EW_TS = 4096
MMA_T = 128
