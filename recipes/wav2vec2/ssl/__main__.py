import sys

from fairseq2_b200.recipe.cli import main

from .recipe import Wav2Vec2SslEvalRecipe, Wav2Vec2SslRecipe

if len(sys.argv) > 1 and sys.argv[1] == "eval":
    sys.exit(main(Wav2Vec2SslEvalRecipe(), sys.argv[2:]))
sys.exit(main(Wav2Vec2SslRecipe()))
