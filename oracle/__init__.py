"""CPU restatement of the reference's FP8 linear path: TEST INFRASTRUCTURE ONLY.

Imported by ``tests/``, by the smoke check and by the CPU-baseline / reference legs of
``bench.py``, as the checker or the timed CPU arm; nothing under ``instinctflash_b200/``
imports it.
"""
