"""Alias of ``skyrl_b200.entrypoints.serve`` under the reference's module path."""

from ...entrypoints.serve import *  # noqa: F401,F403
from ...entrypoints import serve as _impl

if __name__ == "__main__":
    _impl.main()
