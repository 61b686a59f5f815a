"""Hot ops: each module pairs a hand-written sm_100a kernel (through the C ABI of libmstar_kernels.so) with an
fp32 PyTorch oracle that also serves CPU-only runs."""
