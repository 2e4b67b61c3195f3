"""Fused compute + collective kernels over NVLink peer memory, and their host-side plumbing."""
