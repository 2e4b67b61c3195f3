"""Reference arm of the benchmark: runs the unmodified IntelLabs/Optimus-LM code installed under
baseline/_ref for the headline metric.  Prints the same JSON line as bench.py with
``"impl": "reference"``, or ``{"impl": "reference", "unavailable": "<why>"}``."""
import json


def run_reference(opts):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}), flush=True)
