from .base_config import BaseConfig
from .attention import AttnConfig

supported_configs = {
    "attn": AttnConfig,
}
try:
    from .retnet import RetConfig
    from .retnet_bwd import RetBwdConfig
    supported_configs["ret"] = RetConfig
    supported_configs["ret_bwd"] = RetBwdConfig
except ImportError:  # pragma: no cover
    pass
