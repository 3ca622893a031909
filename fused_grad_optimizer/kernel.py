"""Alias of ``forge_b200.kernel`` under the reference package name."""

from forge_b200.kernel import *  # noqa: F401,F403
from forge_b200 import kernel as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
