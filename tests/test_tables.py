"""The generated IQ lookup tables (csrc/kq_iq_tables.inc) are what gguf-py holds."""
from __future__ import annotations

import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def parse(name):
    text = (ROOT / "mlx_kquant_b200" / "csrc" / "kq_iq_tables.inc").read_text()
    body = re.search(name + r"\[\d+\] = \{(.*?)\};", text, re.S).group(1)
    return [int(t, 0) for t in re.findall(r"-?0x[0-9a-fA-F]+|-?\d+", body.replace("ULL", ""))]


def test_tables_have_wire_format_structure():
    ks = parse("kq_tab_ksigns")
    # bit 7 of each sign byte makes the number of minus signs even
    assert all((bin(v).count("1") % 2 == 0) and (v & 127) == i for i, v in enumerate(ks))
    assert parse("kq_tab_kmask") == [1 << j for j in range(8)]
    grid = parse("kq_tab_iq2xxs_grid")
    assert len(grid) == 256 and len(set(grid)) == 256
    assert {(g >> (8 * j)) & 0xFF for g in grid for j in range(8)} == {0x08, 0x19, 0x2B}
    lut = parse("kq_tab_iq4nl")
    assert lut == sorted(lut) and lut[0] == -127 and lut[-1] == 113


def test_tables_match_gguf_py():
    gguf = pytest.importorskip("gguf")
    q = gguf.quants
    assert parse("kq_tab_iq4nl") == [int(v) for v in q.IQ4_NL.kvalues]
    q.IQ2_XXS.init_grid()
    g = np.asarray(q.IQ2_XXS.grid).reshape(256, 8).astype(np.uint8)
    assert parse("kq_tab_iq2xxs_grid") == [int.from_bytes(bytes(r.tolist()), "little") for r in g]
    assert parse("kq_tab_ksigns") == list(q.IQ2_XXS.ksigns)
