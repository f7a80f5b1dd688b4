"""Parity checkers for the Solid GPU path (TEST INFRASTRUCTURE, never shipped).

* ``oracle.ref``          the reference's own Solid CPU library, compiled from the
                          reference checkout by ``oracle/build_ref.py`` into ``oracle/_ref``;
* ``oracle.solid_numpy``  an independent numpy restatement of the same semantics.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this package.
"""
