"""Generates tests/golden/import_block_plan.json: the ExecutionPlan the reference's own LowerRelayToExecPlanPass builds for
the graph of import_block.{json,bin}, serialized by its own SerializeExecutionPlanToJson (oracle/_ref/ref_emit --plan).

Run in a checkout that has the reference compiler built as the checker (make -C oracle ref).
"""
import os
import subprocess

here = os.path.dirname(os.path.abspath(__file__))
root = os.path.dirname(os.path.dirname(here))
emit = os.path.join(root, "oracle", "_ref", "ref_emit")
text = subprocess.run([emit, "--plan", os.path.join(here, "import_block.json"), os.path.join(here, "import_block.bin")],
                      check=True, capture_output=True, text=True).stdout
with open(os.path.join(here, "import_block_plan.json"), "w") as f:
    f.write(text)
print("wrote import_block_plan.json:", len(text), "bytes")
