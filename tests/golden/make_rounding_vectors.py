"""Writes tests/golden/rounding_vectors.json: float64 inputs with their correctly rounded bfloat16 / float16 /
float32 values, computed with exact rational arithmetic (fractions.Fraction), independently of the oracle and of
numpy's casts. Pins `round` of lumen/reference/mod.rs:189-200 (single rounding, ties to even).

Run: python tests/golden/make_rounding_vectors.py
"""

import json
import math
import os
import random
import struct
from fractions import Fraction

FORMATS = {"bfloat16": (8, 7), "float16": (5, 10), "float32": (8, 23)}


def round_exact(x: float, exp_bits: int, man_bits: int) -> float:
    """x rounded to the nearest value of the binary format (ties to even), as a Python float."""
    if math.isnan(x) or math.isinf(x) or x == 0.0:
        return x
    bias = (1 << (exp_bits - 1)) - 1
    emin, emax = 1 - bias, bias
    f = Fraction(abs(x))
    e = math.floor(math.log2(abs(x)))
    while Fraction(2) ** e > f:
        e -= 1
    while Fraction(2) ** (e + 1) <= f:
        e += 1
    e = max(e, emin)
    ulp = Fraction(2) ** (e - man_bits)
    q, r = divmod(f, ulp)
    if r * 2 > ulp or (r * 2 == ulp and q % 2 == 1):
        q += 1
    v = q * ulp
    if v >= Fraction(2) ** (emax + 1):
        return math.copysign(math.inf, x)
    return math.copysign(float(v), x)


def main():
    rng = random.Random(7)
    xs = [0.0, -0.0, 1.0, 1.0 + 2**-8, 1.0 + 2**-8 + 2**-30, 1.0 + 2**-8 - 2**-30, 3.0 + 2**-7, 65504.0, 65519.999,
          65520.0, 2.0**-24, 2.0**-25, 2.0**-25 * 1.0000001, 1.5 * 2.0**-24, 3.3895313892515355e38, 3.4e38, 1e-40, 2.0**-133,
          2.0**-134, 1.0 + 2**-24, 1.0 + 2**-24 + 2**-50, 0.1, 1 / 3, -2.7182818284590451]  # fmt: skip
    for _ in range(400):
        xs.append(struct.unpack("<d", struct.pack("<Q", rng.getrandbits(64)))[0])
    for _ in range(400):
        xs.append(rng.gauss(0, 1) * 10 ** rng.uniform(-6, 6))
    xs = [x for x in xs if not math.isnan(x)]
    out = {"inputs_hex": [x.hex() for x in xs]}
    for name, (e, m) in FORMATS.items():
        out[name] = [float(round_exact(x, e, m)).hex() for x in xs]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rounding_vectors.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print(f"wrote {len(xs)} vectors to {path}")


if __name__ == "__main__":
    main()
