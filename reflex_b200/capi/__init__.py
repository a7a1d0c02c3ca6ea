"""The C interface of the engine: `reflex_b200.h` declares it,
`engine_abi.cpp` implements it over `bridge.py`, `build.py` compiles it into
`libreflex_b200_engine.so`, `client.py` is a Python entry point over it
through ctypes."""
