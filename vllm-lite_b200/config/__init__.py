"""Typed configuration and the architecture registry."""
from .errors import ConfigError, InvalidField, MissingField, UnknownArchitecture  # noqa: F401
from .qwen3 import Qwen3Config, read_config_json  # noqa: F401
from .registry import (ArchitectureEntry, plan_from_config_json, register_architecture,  # noqa: F401
                       registered_architectures, resolve_architecture, unregister_architecture)
from . import qwen3_plan as _qwen3_plan  # noqa: F401  (registers Qwen3ForCausalLM)
from .kikepel import KikepelConfig  # noqa: F401,E402  (registers Kikepel)
from .tuzisun import TuzisunConfig  # noqa: F401,E402  (registers Tuzisun)
from .sodonex import SodonexConfig  # noqa: F401,E402  (registers Sodonex)
from .puturax import PuturaxConfig  # noqa: F401,E402  (registers Puturax)
