from . import tensor
from . import ops
from . import functional
from . import conv
from . import pool
from . import voxelize
