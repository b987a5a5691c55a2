from .safetensors import SafeTensors, SafeTensorsError, load_file, load_file_parallel, save_file
from .tokenizer import BpeTokenizer, Tokenizer, WhitespaceTokenizer, WhitespaceTokenizerConfig

__all__ = ["SafeTensors", "SafeTensorsError", "load_file", "load_file_parallel", "save_file", "BpeTokenizer", "Tokenizer",
           "WhitespaceTokenizer", "WhitespaceTokenizerConfig"]
