"""Utilities: batch packing, sequence bin-packing, stats, tracing, checkpoint helpers."""
