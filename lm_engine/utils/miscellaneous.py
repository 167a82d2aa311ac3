from __future__ import annotations


def divide_if_divisible(dividend: int, divisor: int, msg: str = "") -> int:
    """Exact integer division; raises when ``divisor`` does not divide ``dividend``."""
    if dividend % divisor != 0:
        raise AssertionError(msg or f"{dividend} is not divisible by {divisor}")
    return dividend // divisor


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b
