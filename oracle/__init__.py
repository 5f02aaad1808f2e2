"""CPU checker for the GEMM path. Test infrastructure only: the library never imports it."""
