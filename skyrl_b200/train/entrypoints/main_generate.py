"""Alias of ``skyrl_b200.entrypoints.main_generate`` under the reference's module path."""

from ...entrypoints.main_generate import *  # noqa: F401,F403
from ...entrypoints import main_generate as _impl

if __name__ == "__main__":
    _impl.main()
