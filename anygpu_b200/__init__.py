"""B200-native (sm_100a) Mamba2-mixer forward path behind anyGPU's operator names.

`capi`  - ctypes binding of the C-ABI shared library (the product)
`ops`   - `tensor_<op>` front-end over the ABI for torch-held device memory (imports torch)
`synth` - seeded synthetic weights/inputs of the benchmark configurations (numpy only)
`build` - in-tree nvcc build of the library
"""
__all__ = ["capi", "ops", "synth", "build"]
