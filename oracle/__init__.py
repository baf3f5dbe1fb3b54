"""Checker side of the repository: CPU oracle and the reference's own CUDA build.

Test infrastructure only. Nothing under ``flashgs_b200`` imports this package.
"""
