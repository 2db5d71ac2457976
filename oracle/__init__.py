"""TEST INFRASTRUCTURE: CPU checkers for the MME compute path (not part of the product).

`Port`  -- the plain-C restatement (oracle/mme_oracle.c -> oracle/libmme_oracle.so).
`Ref`   -- the unmodified reference calculator compiled from its own sources
           (oracle/_ref/libmme_ref.so, built by oracle/Makefile where the reference checkout exists).
Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
from .oracle import Port, Ref, build, have_ref  # noqa: F401
