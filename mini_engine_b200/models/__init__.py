"""Architectures.  Importing this package registers the built-in one."""

from mini_engine_b200.models import qwen3  # noqa: F401
