"""CPU checkers for the operator path. TEST INFRASTRUCTURE ONLY.

`oracle.port`  - ctypes binding of libkxc_oracle.so, our plain-C restatement (kxc_oracle.c).
`oracle.ref`   - the unmodified reference compiler's own Relay -> TIR -> C lowering (oracle/_ref/ref_emit),
                 compiled with gcc -ffp-contract=off; the strongest available stand-in for its LLVM
                 CPU backend (LLVM development libraries are not installed in this image).

Only tests/, the smoke check and bench.py's CPU-baseline legs may import this package; the product
(hdkx_aicompiler_b200) never does.
"""
