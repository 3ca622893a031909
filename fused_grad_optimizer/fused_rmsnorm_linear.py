"""Alias of ``forge_b200.rmsnorm_linear`` under the reference package name."""

from forge_b200.rmsnorm_linear import *  # noqa: F401,F403
from forge_b200 import rmsnorm_linear as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
