"""CPU oracle for the tensor-builtin hot path -- test infrastructure, never product code.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
package.  `oracle.binding` loads `libwk_oracle.so` (built by `oracle/Makefile`).
"""
