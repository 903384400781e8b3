"""Stand-in for the reference's CPU module ``fixed_extension`` (torch_c/sc-extension/fixed.cpp:240-242); imported
by the front end (utils_functional.py:19), never called.  No CPU arithmetic is shipped."""


def conv2d_saturate(*args, **kwargs):
    raise NotImplementedError(
        "fixed_extension.conv2d_saturate: rexsc_b200 has no CPU implementation; use fixed_extension_cuda")
