"""Integer helpers (reference: spio/util/math.py)."""

from math import gcd


def divup(n: int, d: int) -> int:
    """Ceiling of n / d."""
    return -(-n // d)


def next_relative_prime(n: int, modulus: int) -> int:
    """Smallest integer >= n that shares no factor with modulus."""
    while gcd(n, modulus) != 1:
        n += 1
    return n
