"""CPU oracle for the trinix_b200 parity tests (test infrastructure, never shipped).

Only tests/, the smoke run and the benchmark's CPU-baseline / reference legs may
import from here.
"""
