import sys

from fairseq2_b200.recipe.cli import main

from .recipe import Wav2Vec2AsrEvalRecipe, Wav2Vec2AsrRecipe

if len(sys.argv) > 1 and sys.argv[1] == "eval":
    sys.exit(main(Wav2Vec2AsrEvalRecipe(), sys.argv[2:]))
sys.exit(main(Wav2Vec2AsrRecipe()))
