"""CPU oracle for the training-step hot path.  TEST INFRASTRUCTURE ONLY: imported by tests/,
``__graft_entry__.smoke()`` and the CPU arms of ``bench.py`` — never by ``tinyflow_b200``."""
