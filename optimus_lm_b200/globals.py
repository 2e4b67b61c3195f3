"""Process-wide handles.  ``profiler`` is the active ``PclProfiler`` or ``None``
(reference optimus/globals.py:1)."""
profiler = None
