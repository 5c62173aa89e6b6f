"""Old import paths of the reference (CodeGen.runner, CodeGen.gemmini, ...) kept as aliases."""
