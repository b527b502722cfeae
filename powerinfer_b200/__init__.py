"""B200 (sm_100a) implementation of PowerInfer's decode hot path.

`ggml_ops` and `engine` call the CUDA library through its C ABI and raise ImportError when
libpowerinfer_b200.so has not been built (`python -m powerinfer_b200.build`); there is no CPU or
eager-torch fallback.  `synth` and `build` are host-only helpers and import without it.
"""
