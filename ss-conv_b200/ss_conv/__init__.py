"""ss_conv — sparse steerable convolution layers backed by the B200 CUDA library.

Same public layout as the reference package (SS_Conv_lib/ss_conv/__init__.py).
"""
from . import _ext
from . import sp_ops
from . import utils

from . import convolution
from . import activation
from . import batchnorm
from . import pool
from . import dropout
from . import parallel
