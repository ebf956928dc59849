"""Peer memory, tensor parallelism and prefill/decode disaggregation."""
