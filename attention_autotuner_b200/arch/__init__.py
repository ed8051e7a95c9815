from .arch_base import Arch
from .A100 import *
from .RTX4090 import *
from .B200 import *
