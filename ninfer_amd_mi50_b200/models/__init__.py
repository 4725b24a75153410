from . import qwen2_moe  # noqa: F401  (registration)
