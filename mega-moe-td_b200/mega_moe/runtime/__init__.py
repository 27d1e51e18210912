"""Symmetric workspaces and routing metadata (mirrors src/mega_moe/runtime of the reference)."""
