"""pluto_b200: a B200-native (sm_100a) attention engine behind Pluto's layer interface.

`pluto_b200.layers` mirrors the reference's layer classes; `pluto_b200._capi` binds the C ABI of
include/pluto_b200.h; the kernels live in `pluto_b200/csrc`.
"""
from ._capi import PlutoStatusError  # noqa: F401
