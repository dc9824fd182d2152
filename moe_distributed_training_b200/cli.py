"""Keyword-argument command line in the style of python-fire.

The reference exposes every keyword of `main()` as a `--flag value` option through
`fire.Fire(main)` (train_accelerate_fsdp2.py:473-475).  `fire` is not a dependency
here; this does the same from the function signature: `--flag value`,
`--flag=value`, bare `--flag` for booleans, with types taken from the defaults.
"""
from __future__ import annotations

import inspect
import sys
from typing import Callable, List, Optional


def _convert(text: str, default, annotation):
    low = text.lower()
    if isinstance(default, bool) or annotation is bool:
        if low in ("true", "1", "yes"):
            return True
        if low in ("false", "0", "no"):
            return False
        raise ValueError(f"expected a boolean, got '{text}'")
    if low in ("none", "null"):
        return None
    for typ in ((type(default),) if default is not None else ()) + (int, float):
        if typ in (int, float):
            try:
                return typ(text)
            except ValueError:
                continue
        if typ is str:
            return text
    return text


def parse_kwargs(fn: Callable, argv: List[str]) -> dict:
    sig = inspect.signature(fn)
    out, i = {}, 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--"):
            raise SystemExit(f"unexpected argument '{tok}' (flags look like --name value)")
        name, eq, val = tok[2:].partition("=")
        name = name.replace("-", "_")
        if name not in sig.parameters:
            raise SystemExit(f"unknown flag --{name}; known flags: {', '.join(sig.parameters)}")
        par = sig.parameters[name]
        if not eq:
            nxt = argv[i + 1] if i + 1 < len(argv) else None
            if nxt is None or nxt.startswith("--"):
                val = "true"
            else:
                val, i = nxt, i + 1
        out[name] = _convert(val, par.default if par.default is not inspect._empty else None, par.annotation)
        i += 1
    return out


def run(fn: Callable, argv: Optional[List[str]] = None):
    return fn(**parse_kwargs(fn, sys.argv[1:] if argv is None else argv))
