"""Alias of ``forge_b200.state`` under the reference package name."""

from forge_b200.state import *  # noqa: F401,F403
from forge_b200 import state as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
