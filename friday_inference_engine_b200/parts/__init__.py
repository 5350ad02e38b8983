"""Parts that layers are put together from.  Importing this package registers the
parts that the library ships; a caller registers more with `register_part`."""
from .base import (BuildEnv, KVRequest, Param, Part, StateRequest, build_part,  # noqa: F401
                   register_part)
from .spec import LayerCall, ModelSpec, PartSpec  # noqa: F401
from . import attention, block, mlp, norm, rotary  # noqa: F401,E402
