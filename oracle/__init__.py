"""CPU oracle for the grouped-GEMM path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``grouped_gemm_b200/`` imports this package; only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` do, as the checker or as the timed CPU baseline.
"""
