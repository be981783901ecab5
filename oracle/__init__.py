"""CPU oracle for the JetFire decode hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``jetfire_b200/`` may import this
package; only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference arms of ``bench.py`` do, and only as the checker or the timed CPU
baseline -- never as the product path.
"""
