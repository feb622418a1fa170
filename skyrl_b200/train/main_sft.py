"""Alias of ``skyrl_b200.entrypoints.main_sft`` under the reference's module path (``<pkg>.train.main_sft``)."""

from ..entrypoints.main_sft import *  # noqa: F401,F403
from ..entrypoints import main_sft as _impl

if __name__ == "__main__":
    _impl.main()
