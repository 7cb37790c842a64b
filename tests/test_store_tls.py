"""TLS 1.3 on the config-store links (mutual certificate verification, OpenSSL opened at run time): a store served and used
over TLS, and the refusals: a plaintext client, a certificate from another CA, a revoked certificate, a wrong pass phrase."""
import datetime
import os

import pytest

import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402
import memfabric_hybrid_b200.api as mf

crypto = pytest.importorskip("cryptography")
from cryptography import x509  # noqa: E402
from cryptography.hazmat.primitives import hashes, serialization  # noqa: E402
from cryptography.hazmat.primitives.asymmetric import ec  # noqa: E402
from cryptography.x509.oid import NameOID  # noqa: E402


def _name(cn):
    return x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, cn)])


def _now():
    return datetime.datetime.now(datetime.timezone.utc)


def _make_ca(cn):
    key = ec.generate_private_key(ec.SECP256R1())
    cert = (x509.CertificateBuilder().subject_name(_name(cn)).issuer_name(_name(cn)).public_key(key.public_key())
            .serial_number(x509.random_serial_number()).not_valid_before(_now() - datetime.timedelta(days=1))
            .not_valid_after(_now() + datetime.timedelta(days=365))
            .add_extension(x509.BasicConstraints(ca=True, path_length=None), critical=True)
            .add_extension(x509.KeyUsage(digital_signature=True, key_cert_sign=True, crl_sign=True, content_commitment=False,
                                         key_encipherment=False, data_encipherment=False, key_agreement=False,
                                         encipher_only=False, decipher_only=False), critical=True)
            .sign(key, hashes.SHA256()))
    return key, cert


def _make_leaf(ca_key, ca_cert, cn):
    key = ec.generate_private_key(ec.SECP256R1())
    cert = (x509.CertificateBuilder().subject_name(_name(cn)).issuer_name(ca_cert.subject).public_key(key.public_key())
            .serial_number(x509.random_serial_number()).not_valid_before(_now() - datetime.timedelta(days=1))
            .not_valid_after(_now() + datetime.timedelta(days=90))
            .add_extension(x509.BasicConstraints(ca=False, path_length=None), critical=True)
            .sign(ca_key, hashes.SHA256()))
    return key, cert


def _pem_cert(c):
    return c.public_bytes(serialization.Encoding.PEM)


def _pem_key(k, password=None):
    enc = serialization.BestAvailableEncryption(password) if password else serialization.NoEncryption()
    return k.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.PKCS8, enc)


@pytest.fixture(scope="module")
def pki(tmp_path_factory):
    d = tmp_path_factory.mktemp("pki")
    ca_key, ca = _make_ca("mf test CA")
    other_key, other = _make_ca("some other CA")
    files = {"ca.pem": _pem_cert(ca), "other_ca.pem": _pem_cert(other)}
    for who, (k, c) in {"node": _make_leaf(ca_key, ca, "node"), "revoked": _make_leaf(ca_key, ca, "revoked"),
                        "stranger": _make_leaf(other_key, other, "stranger")}.items():
        files[who + ".crt"] = _pem_cert(c)
        files[who + ".key"] = _pem_key(k)
        if who == "node":
            files["node_enc.key"] = _pem_key(k, b"s3cret-phrase")
        if who == "revoked":
            rc = x509.RevokedCertificateBuilder().serial_number(c.serial_number).revocation_date(_now()).build()
            crl = (x509.CertificateRevocationListBuilder().issuer_name(ca.subject).last_update(_now() - datetime.timedelta(hours=1))
                   .next_update(_now() + datetime.timedelta(days=30)).add_revoked_certificate(rc).sign(ca_key, hashes.SHA256()))
            files["crl.pem"] = crl.public_bytes(serialization.Encoding.PEM)
    for n, b in files.items():
        (d / n).write_bytes(b)
    (d / "pass.txt").write_text("s3cret-phrase\n")
    return d


def _info(d, cert="node.crt", key="node.key", ca="ca.pem", crl=None, pwd=None):
    s = f"tlsCaPath: {d}/; tlsCaFile: {ca}; tlsCert: {d}/{cert}; tlsPk: {d}/{key}"
    if crl:
        s += f"; tlsCrlPath: {d}/; tlsCrlFile: {crl}"
    if pwd:
        s += f"; tlsPkPwd: {d}/{pwd}"
    return s


@pytest.fixture()
def tls_off():
    yield
    mf.set_conf_store_tls(False, "")
    H.lib().smem_set_config_store_tls_key(None, 0, None, 0, None)  # forget any key given through the key call


def test_store_over_tls(pki, tls_off):
    assert mf.set_conf_store_tls(True, _info(pki)) == 0
    port = free_port()
    srv = H.start_server(port, world=4)
    try:
        a, b = H.Store.connect(port, rank=0), H.Store.connect(port, rank=1)
        assert a.set("k", b"over tls") == 0 and b.get("k") == b"over tls"
        # the periodic certificate check, run by hand: the leaf certificates of this test are valid for 90 days
        check = H.lib().mf_t_tls_check_now
        check.restype = H.C.c_int
        assert 85 <= check() <= 90
        big = os.urandom(3 << 20)   # several TLS records and more than one socket buffer
        assert a.set("big", big) == 0 and b.get("big", cap=4 << 20) == big
        assert b.add("n", 7) == 7
        # a plaintext client is turned away during the handshake
        mf.set_conf_store_tls(False, "")
        with pytest.raises(ConnectionError):
            H.Store.connect(port, rank=2, timeout_ms=1500)
        # so is a client whose certificate was issued by another CA
        assert mf.set_conf_store_tls(True, _info(pki, cert="stranger.crt", key="stranger.key")) == 0
        with pytest.raises(ConnectionError):
            H.Store.connect(port, rank=2, timeout_ms=1500)
        # the links that were up keep working
        assert a.get("k") == b"over tls"
        a.close()
        b.close()
    finally:
        H.lib().mf_t_server_stop(srv)


def test_revoked_certificate_is_refused(pki, tls_off):
    assert mf.set_conf_store_tls(True, _info(pki, crl="crl.pem")) == 0
    port = free_port()
    srv = H.start_server(port, world=4)
    try:
        ok = H.Store.connect(port, rank=0)
        assert ok.set("x", b"1") == 0
        assert mf.set_conf_store_tls(True, _info(pki, cert="revoked.crt", key="revoked.key", crl="crl.pem")) == 0
        with pytest.raises(ConnectionError):
            H.Store.connect(port, rank=1, timeout_ms=1500)
        ok.close()
    finally:
        H.lib().mf_t_server_stop(srv)


def test_encrypted_key_and_the_key_call(pki, tls_off):
    # pass phrase from a file named in the info string
    assert mf.set_conf_store_tls(True, _info(pki, key="node_enc.key", pwd="pass.txt")) == 0
    port = free_port()
    srv = H.start_server(port, world=4)
    try:
        c = H.Store.connect(port, rank=0)
        assert c.set("k", b"v") == 0
        c.close()
    finally:
        H.lib().mf_t_server_stop(srv)
    # key as PEM text through the key call, pass phrase "encrypted" by reversal and handed to a Python decrypter
    info = f"tlsCaPath: {pki}/; tlsCaFile: ca.pem; tlsCert: {pki}/node.crt"
    assert mf.set_conf_store_tls(True, info) == 0
    pem = (pki / "node_enc.key").read_text()
    assert mf.set_conf_store_tls_key(pem, "esarhp-terc3s", lambda s: s[::-1]) == 0
    port = free_port()
    srv = H.start_server(port, world=4)
    try:
        c = H.Store.connect(port, rank=0)
        assert c.set("k2", b"v2") == 0 and c.get("k2") == b"v2"
        c.close()
    finally:
        H.lib().mf_t_server_stop(srv)
    # a wrong pass phrase: the store refuses to start instead of falling back to plaintext
    assert mf.set_conf_store_tls_key(pem, "wrong") == 0
    rc = H.C.c_int()
    assert not H.lib().mf_t_server_start(b"127.0.0.1", free_port(), 4, 0, H.C.byref(rc)) and rc.value != 0


def test_bad_tls_info_is_rejected(tls_off):
    assert mf.set_conf_store_tls(True, "tlsCert /nowhere") != 0
    assert mf.set_conf_store_tls(True, "bogusKey: 1; tlsCert: /x; tlsCaPath: /y") != 0
    assert mf.set_conf_store_tls(True, "tlsCaPath: /y") != 0
