import sys

from fairseq2_b200.recipe.cli import main

from .recipe import LMTrainRecipe

sys.exit(main(LMTrainRecipe()))
