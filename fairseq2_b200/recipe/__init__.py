from fairseq2_b200.recipe.base import (EvalRecipe, GenerationRecipe, Recipe, RecipeContext, RecipeDataset,
                                       RecipeModel, RecipeTokenizer, TrainRecipe)
from fairseq2_b200.recipe.cli import main
from fairseq2_b200.recipe.run import load_recipe_config, run_recipe
