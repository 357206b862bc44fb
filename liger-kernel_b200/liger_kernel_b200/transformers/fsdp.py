"""Run a function from inside an FSDP-wrapped module's ``forward`` so that the module's full
parameters are gathered while it runs (reference: ``src/liger_kernel/transformers/fsdp.py:7-55``)."""


def run_inside_fsdp_forward(wrapper_module, fn, *args, **kwargs):
    inner = wrapper_module._fsdp_wrapped_module if hasattr(wrapper_module, "_fsdp_wrapped_module") else wrapper_module.module
    original_forward = inner.forward

    def redirected(*_a, **_k):
        inner.forward = original_forward  # restore first: fn may call the real forward
        return fn(*args, **kwargs)

    inner.forward = redirected
    try:
        return wrapper_module()
    finally:
        inner.forward = original_forward
