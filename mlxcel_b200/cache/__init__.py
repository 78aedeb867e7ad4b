from .kv_pool import KVPool  # noqa: F401
