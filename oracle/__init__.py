"""CPU checkers for the tests and the benchmark's CPU leg; never imported by the package."""
