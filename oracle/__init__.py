"""CPU checker for the Conv2d path. Test infrastructure only: imported by tests/, by the smoke
check and by the CPU-baseline leg of bench.py, never by the tracea_b200 package."""
