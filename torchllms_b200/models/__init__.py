"""Architectures: each module registers one family with the architecture registry."""
