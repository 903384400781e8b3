"""Drop-in for the reference's ``sc_extension_cuda`` pybind module (torch_c/sc-extension/sc_cuda.cpp:122-132):
same nine functions, same positional arguments, backed by librexsc_b200.so."""
from rexsc_b200.ops import (  # noqa: F401
    conv2d_generic_general_acc,
    conv2d_generic_general_split_acc,
    linear_generic_general_acc,
    or_approx_n_backward_acc,
    or_approx_n_backward_bias_std_acc,
    or_approx_n_backward_bias_std_both_acc,
    or_approx_n_forward_acc,
    or_approx_n_forward_bias_std_acc,
    or_approx_n_forward_bias_std_both_acc,
)
