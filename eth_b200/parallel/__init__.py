"""Parallel runtime: process-group registry, tensor-parallel layers, resharding, gradient sync."""
