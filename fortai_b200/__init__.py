"""B200 (sm_100a) Q8_0 matvec / prefill backend behind FortAI's CUDA C ABI.

`fortai_b200.abi` loads the shared library and declares every exported symbol;
`fortai_b200.backend_cuda` mirrors the reference's Fortran wrapper module
(src/backend/cuda/fortai_backend_cuda.f90) on top of it; `fortai_b200.sharded`
holds the row / column sharding used across the GPUs of one box.

There is no CPU fallback: importing `abi` fails when the library cannot be
built or loaded.
"""
__all__ = ["abi", "backend_cuda", "build", "sharded"]
