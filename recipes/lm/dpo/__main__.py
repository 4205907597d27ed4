import sys

from fairseq2_b200.recipe.cli import main

from .recipe import LMDPORecipe

sys.exit(main(LMDPORecipe()))
