"""Architecture modules.  Importing this package registers every architecture
the library knows; a new one is a new module here that calls
`register_architecture`."""

from . import qwen3  # noqa: F401
