"""Drop-in for the reference's ``fixed_extension_cuda`` pybind module (torch_c/sc-extension/fixed_cuda.cpp:36-38)."""
from rexsc_b200.ops import conv2d_saturate_acc  # noqa: F401
