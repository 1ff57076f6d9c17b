"""TEST INFRASTRUCTURE - CPU oracle of the fused-MoE path.

Nothing in the product imports this package.  It is used by ``tests/``, by the
smoke check and by the CPU-baseline leg of ``bench.py`` only.
"""
