"""CPU oracle for the Q4_0 x Q8_1 path: test infrastructure, not part of the shipped library.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark import this
package.  See ``jq_oracle.c`` for the arithmetic and ``jq_oracle.py`` for the loader and the
independent NumPy mirror.
"""
