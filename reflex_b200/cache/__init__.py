from .specs import KVSpec, StateSpec  # noqa: F401
from .pool import IdPool  # noqa: F401
from .store import PAGE_TOKENS, Cache, KVGroup, KVView, StateGroup  # noqa: F401
