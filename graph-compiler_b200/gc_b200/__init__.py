"""gc_b200 — host-side Python mirror of the B200 backend for Intel Graph Compiler partitions."""
