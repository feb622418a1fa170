"""Module paths of the reference (``<pkg>.train.entrypoints.{main_base,main_generate,serve}``) for launch lines and
imports that were written against it; the implementations live in ``skyrl_b200.entrypoints``."""
