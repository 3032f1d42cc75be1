"""Fused compute + collective kernels over NVLink peer memory and the symmetric-memory runtime they use."""
