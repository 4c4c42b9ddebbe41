"""TEST INFRASTRUCTURE ONLY: a plain-Python restatement of rllama's tokenizer (``src/tokenizer.rs``),
used by the tests to check the library's C++ tokenizer. Nothing shipped imports this file.

The piece table comes from the ``sentencepiece`` package's own reading of the model file, so the
library's protobuf reader is checked against an independent parser. PARITY UNPINNED against the Rust
binary itself (no Rust toolchain and no ``tokenizer.model`` golden strings in the reference tree).
"""


def load_pieces(model_bytes):
    """``Tokenizer::load`` (``src/tokenizer.rs:46-96``): text -> index; later duplicates win."""
    import sentencepiece as spm

    sp = spm.SentencePieceProcessor(model_proto=model_bytes)
    pieces = {}
    for idx in range(sp.get_piece_size()):
        pieces[sp.id_to_piece(idx)] = idx
    return pieces


def tokenize_to_pieces(pieces, s):
    """``Tokenizer::tokenize_to_pieces`` (``src/tokenizer.rs:125-164``): scan every piece, keep the
    longest one (in bytes) that prefixes the rest of the text."""
    result = []
    while s:
        best, best_len, skip = "", 0, ""
        if s.startswith("\n"):
            if "<0x0A>" in pieces:
                best, best_len, skip = "<0x0A>", len("<0x0A>"), s[1:]
        else:
            for piece in sorted(pieces):  # BTreeMap order
                blen = len(piece.encode("utf-8"))
                if s.startswith(piece) and best_len < blen:
                    best, best_len, skip = piece, blen, s[len(piece):]
        if best_len == 0:
            # str::get(1..): None unless byte 1 is a character boundary (src/tokenizer.rs:153-155)
            raw = s.encode("utf-8")
            if len(raw) > 1 and (raw[1] & 0xC0) == 0x80:
                s = ""
            else:
                s = raw[1:].decode("utf-8")
        else:
            result.append(best)
            s = skip
    return result


def tokenize_to_ids(pieces, text):
    """``Tokenizer::tokenize_to_ids`` (``src/tokenizer.rs:166-178``)."""
    s = ("▁" + text).replace(" ", "▁")
    return [1] + [pieces[p] for p in tokenize_to_pieces(pieces, s)]
