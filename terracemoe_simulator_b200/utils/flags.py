"""Environment switches, parsed strictly: an unknown value raises instead of silently meaning
"off" (the rule of the reference's flag system: new capability defaults off, unknown values
raise; ``terrace/ta2a_pack.py:114-143``).

    flag_bool("TERRACE_EP_OVERLAP", True)         -> True unless set to 0 / off / false / no
    flag_choice("TERRACE_ATTENTION", ("native", "sdpa"), "native")
    check_native_flags()                           -> validates the switches the C++ side reads
"""
from __future__ import annotations

import os

_TRUE = ("1", "on", "true", "yes")
_FALSE = ("0", "off", "false", "no", "")


def flag_bool(name: str, default: bool = False) -> bool:
    raw = os.environ.get(name)
    if raw is None:
        return default
    v = raw.strip().lower()
    if v in _TRUE:
        return True
    if v in _FALSE:
        return False
    raise ValueError(f"{name}={raw!r}: expected one of {_TRUE + _FALSE[:-1]}")


def flag_choice(name: str, choices, default: str) -> str:
    raw = os.environ.get(name)
    if raw is None or raw.strip() == "":
        return default
    v = raw.strip().lower()
    if v not in choices:
        raise ValueError(f"{name}={raw!r}: expected one of {tuple(choices)}")
    return v


def flag_int(name: str, default: int, lo: int, hi: int) -> int:
    raw = os.environ.get(name)
    if raw is None or raw.strip() == "":
        return default
    try:
        v = int(raw.strip())
    except ValueError:
        raise ValueError(f"{name}={raw!r}: expected an integer in [{lo}, {hi}]") from None
    if not lo <= v <= hi:
        raise ValueError(f"{name}={raw!r}: expected an integer in [{lo}, {hi}]")
    return v


def check_native_flags() -> None:
    """The switches that the native library reads with ``getenv``; validated here, once, when the
    library is loaded, because C++ has nobody to raise to."""
    flag_choice("TERRACE_GEMM_PAIR", ("0", "1", "auto"), "auto")
