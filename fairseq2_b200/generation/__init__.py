from fairseq2_b200.generation.generator import (BeamSearchAlgorithm, BeamSearchSequenceGenerator, Hypothesis,
                                                SamplingSequenceGenerator, SequenceGenerator,
                                                SequenceGeneratorOutput, StandardBeamSearchAlgorithm)
from fairseq2_b200.generation.sampler import Sampler, TopKSampler, TopPSampler
from fairseq2_b200.generation.step_processor import (BannedSequenceProcessor, NGramRepeatBlockProcessor,
                                                     StepProcessor)
from fairseq2_b200.generation.seq2seq import (BeamSearchSeq2SeqGenerator, SamplingSeq2SeqGenerator,
                                              Seq2SeqGenerator)
from fairseq2_b200.generation.text import SequenceToTextConverter, TextCompleter, TextTranslator
