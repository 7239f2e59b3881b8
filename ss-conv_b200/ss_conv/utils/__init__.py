from . import utils
from . import SO3
from . import kernel
