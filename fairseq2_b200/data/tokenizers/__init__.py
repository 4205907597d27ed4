from fairseq2_b200.data.tokenizers.char import CharTokenizer
from fairseq2_b200.data.tokenizers.hub import load_tokenizer, register_tokenizer_family
from fairseq2_b200.data.tokenizers.tokenizer import TokenDecoder, TokenEncoder, Tokenizer, VocabularyInfo
