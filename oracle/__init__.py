"""CPU oracle of the encoder hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only ``tests/``, the
smoke check and the CPU-baseline leg of ``bench.py`` may import it.  Every
function restates the arithmetic of the reference's fp32 torch path and cites
the reference file:line it follows.
"""
