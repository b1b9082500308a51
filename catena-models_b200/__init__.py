"""A small B200-native generation library for the LFM3 hybrid decoder of catena-models:
typed configuration and an architecture registry, safetensors weights by name, layers put
together from parts, a paged cache with a slot per sequence, one batched step function, a
generation loop with greedy and temperature sampling, and hand-written sm_100a kernels.
"""
from .config.base import ConfigError  # noqa: F401
from .config.registry import architectures, register_architecture  # noqa: F401
from .parts import build_part, register_part  # noqa: F401
from . import models as _models  # noqa: F401  (registers the built-in architecture)


def __getattr__(name):
    # The API classes need torch.cuda at use time only; importing the package stays light.
    if name in ("Model", "Session"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
