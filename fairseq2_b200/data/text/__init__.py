from fairseq2_b200.data.text.converters import StrSplitter, StrToIntConverter, StrToTensorConverter
from fairseq2_b200.data.text.reader import LineEnding, read_text
