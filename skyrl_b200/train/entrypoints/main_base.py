"""Alias of ``skyrl_b200.entrypoints.main_base`` under the reference's module path."""

from ...entrypoints.main_base import *  # noqa: F401,F403
from ...entrypoints import main_base as _impl

if __name__ == "__main__":
    _impl.main()
