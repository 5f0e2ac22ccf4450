"""Adapters that plug the compressed KV path into serving engines."""
