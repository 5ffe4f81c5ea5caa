"""Test helpers: the oracle glue lives with the oracle (test infrastructure)."""

from oracle.torch_glue import (  # noqa: F401
    ORACLE_DTYPE,
    TOLERANCE,
    assert_close,
    bits,
    from_bits,
    oracle_decode,
    oracle_rope_write,
    same_bits,
)
