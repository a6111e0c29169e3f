"""Pixels -> patches -> merged vision tokens for the sweep's image sizes (reference:
scripts/compute_vision_tokens.py:15-71)."""
from __future__ import annotations

import argparse

SWEEP_SIDES = (448, 896, 1344, 1792, 2240, 3584)


def vision_tokens(side: int, patch: int = 14, merge: int = 2) -> dict:
    g = side // patch
    g -= g % merge
    patches = g * g
    return {"side": side, "pixels": side * side, "grid": g, "patches": patches, "merged_tokens": patches // merge ** 2,
            "windows": (-(-(g // merge) // 4)) ** 2}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sides", type=int, nargs="*", default=list(SWEEP_SIDES))
    a = ap.parse_args(argv)
    print(f"{'side':>6} {'pixels':>10} {'patches':>8} {'merged':>8} {'windows':>8}")
    for s in a.sides:
        r = vision_tokens(s)
        print(f"{r['side']:>6} {r['pixels']:>10} {r['patches']:>8} {r['merged_tokens']:>8} {r['windows']:>8}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
