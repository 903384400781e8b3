"""Stand-in for the reference's CPU module ``sc_extension`` (torch_c/sc-extension/sc.cpp:34-37).  The front end
imports it (utils_functional.py:17) and never calls it; this library ships no CPU arithmetic, so the functions
exist only to fail loudly if something does call them."""


def _no_cpu_path(name):
    def fn(*args, **kwargs):
        raise NotImplementedError(
            f"sc_extension.{name}: rexsc_b200 has no CPU implementation; use sc_extension_cuda on a CUDA device")
    fn.__name__ = name
    return fn


conv2d_generic_general = _no_cpu_path("conv2d_generic_general")
linear_generic_general = _no_cpu_path("linear_generic_general")
