"""Reference arm of bench.py: runs the unmodified reference trainer from baseline/_ref."""
import json


def run_reference_arm(args) -> dict:
    return {"impl": "reference", "unavailable": "reference install not set up yet"}
