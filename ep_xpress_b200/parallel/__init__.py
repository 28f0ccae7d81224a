"""Transports and their runtime: control plane, peer-mapped heap, contexts."""
