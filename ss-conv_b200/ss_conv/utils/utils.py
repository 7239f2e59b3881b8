"""Small helpers shared by the layers (interface of SS_Conv_lib/ss_conv/utils/utils.py)."""
import torch


def Rs2dim(Rs):
    """Number of channels of a list of (multiplicity, order) pairs."""
    return sum(m * (2 * l + 1) for m, l in Rs)


def calculate_fan_in(channel_in, kernel_size):
    fan = channel_in
    for k in kernel_size:
        fan *= int(k)
    return fan


class torch_default_dtype:
    """Context manager that temporarily switches torch's default dtype."""

    def __init__(self, dtype):
        self.dtype = dtype
        self.saved = None

    def __enter__(self):
        self.saved = torch.get_default_dtype()
        torch.set_default_dtype(self.dtype)

    def __exit__(self, exc_type, exc_value, traceback):
        torch.set_default_dtype(self.saved)
