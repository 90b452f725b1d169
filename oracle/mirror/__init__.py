"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: the reference's call sites above the backend trait, restated in Python.

`tensor` follows crates/weta-tensor/src/tensor.rs, `autograd` crates/weta-autograd/src/ops.rs and graph.rs, `nn`
crates/weta-nn/src/{functional,layers}.rs and crates/weta-optim/src/lib.rs, `models` the named models and their
training step (crates/weta/examples/mnist_{mlp,cnn}.rs).  They issue, primitive by primitive, the backend-call stream
the reference issues, against any object with the backend method set: the CPU oracle (`oracle.cpu_backend`) to obtain
expected values, or the CUDA backend to exercise the trait entry points.  Only tests, `smoke()` and the benchmark's
CPU-baseline leg import this package; nothing under `weta_b200/` does.
"""
