"""Import-name shim: the reference's scripts do ``from eed.backend import ...``
(script/benchmark.py:3, script/standard-test.py:3-7)."""
