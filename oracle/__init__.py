"""CPU oracle for the BaM hot path.  Test infrastructure: imported by tests/, smoke() and the
cpu_baseline / reference arm of bench.py only -- never by the bam_b200 package."""
