"""Command-line helpers that ship with the engine (``python -m lmms_engine_b200.tools.<name>``)."""
