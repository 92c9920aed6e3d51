"""Baseline harness: runs the unmodified reference (installed under ``baseline/_ref``) for the
headline benchmark. Nothing in here is imported by the ``ohara_b200`` package."""
