"""CPU oracle (test infrastructure).  Only the tests, the smoke check and the
benchmark's CPU-baseline leg import this package; the shipped library never does."""
