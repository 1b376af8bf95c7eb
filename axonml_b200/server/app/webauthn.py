"""WebAuthn (FIDO2) second factor for the platform server: registration and assertion ceremonies
with ES256 credentials, verified on the server as the W3C WebAuthn Level 2 text prescribes
(client data type / challenge / origin, relying-party id hash, user-present flag, signature over
``authenticatorData || SHA-256(clientDataJSON)``, signature counter).

The wire shapes are the reference's (crates/axonml-server/src/auth/webauthn.rs:13-141:
``RegistrationChallenge``, ``AuthenticationChallenge``, ``RegistrationResponse``,
``AuthenticationResponse``, ``WebAuthnCredential``; its finish_* functions, :201-296, accept
whatever the client sends and do not check a signature).  Attestation formats ``none`` and
``packed`` self-attestation are accepted; a certificate chain is not evaluated (the server asks
for ``attestation: "none"``).  Binary fields travel as unpadded base64url.

Signature checks use the ``cryptography`` package; without it ``available()`` is False and the
routes answer 501."""
from __future__ import annotations

import base64
import hashlib
import json
import os
import time

ES256 = -7


def available() -> bool:
    try:
        import cryptography.hazmat.primitives.asymmetric.ec  # noqa: F401
        return True
    except Exception:          # pragma: no cover - depends on the image
        return False


class WebAuthnError(ValueError):
    pass


def b64u(data: bytes) -> str:
    return base64.urlsafe_b64encode(data).rstrip(b"=").decode()


def b64u_dec(text: str) -> bytes:
    text = text.strip().replace("+", "-").replace("/", "_")
    return base64.urlsafe_b64decode(text + "=" * (-len(text) % 4))


# ---------------------------------------------------------------------------------- CBOR (RFC 8949 subset)
def cbor_decode(data: bytes, pos: int = 0):
    """Decodes one item of the subset authenticators use (ints, byte / text strings, arrays, maps,
    false / true / null); returns ``(value, next_pos)``."""
    if pos >= len(data):
        raise WebAuthnError("truncated CBOR")
    ib = data[pos]
    major, info = ib >> 5, ib & 31
    pos += 1
    if info < 24:
        val = info
    elif info in (24, 25, 26, 27):
        n = 1 << (info - 24)
        if pos + n > len(data):
            raise WebAuthnError("truncated CBOR")
        val = int.from_bytes(data[pos:pos + n], "big")
        pos += n
    else:
        raise WebAuthnError("unsupported CBOR length form")
    if major == 0:
        return val, pos
    if major == 1:
        return -1 - val, pos
    if major in (2, 3):
        if pos + val > len(data):
            raise WebAuthnError("truncated CBOR")
        raw = data[pos:pos + val]
        return (bytes(raw) if major == 2 else raw.decode("utf-8")), pos + val
    if major == 4:
        out = []
        for _ in range(val):
            item, pos = cbor_decode(data, pos)
            out.append(item)
        return out, pos
    if major == 5:
        out = {}
        for _ in range(val):
            k, pos = cbor_decode(data, pos)
            v, pos = cbor_decode(data, pos)
            out[k] = v
        return out, pos
    if major == 7 and info in (20, 21, 22):
        return {20: False, 21: True, 22: None}[info], pos
    raise WebAuthnError("unsupported CBOR item")


def cbor_encode(obj) -> bytes:
    """The same subset, for building attestation objects (tests, software authenticators)."""
    def head(major: int, n: int) -> bytes:
        if n < 24:
            return bytes([major << 5 | n])
        for info, size in ((24, 1), (25, 2), (26, 4), (27, 8)):
            if n < 1 << (8 * size):
                return bytes([major << 5 | info]) + n.to_bytes(size, "big")
        raise WebAuthnError("integer too large for CBOR")
    if obj is False or obj is True or obj is None:
        return bytes([0xE0 | {False: 20, True: 21, None: 22}[obj]])
    if isinstance(obj, int):
        return head(0, obj) if obj >= 0 else head(1, -1 - obj)
    if isinstance(obj, (bytes, bytearray)):
        return head(2, len(obj)) + bytes(obj)
    if isinstance(obj, str):
        raw = obj.encode("utf-8")
        return head(3, len(raw)) + raw
    if isinstance(obj, (list, tuple)):
        return head(4, len(obj)) + b"".join(cbor_encode(x) for x in obj)
    if isinstance(obj, dict):
        return head(5, len(obj)) + b"".join(cbor_encode(k) + cbor_encode(v) for k, v in obj.items())
    raise WebAuthnError(f"cannot encode {type(obj).__name__} as CBOR")


# ---------------------------------------------------------------------------------- authenticator data
def parse_authenticator_data(data: bytes) -> dict:
    """rpIdHash (32) | flags (1) | signCount (4) | [attested credential data] | [extensions]."""
    if len(data) < 37:
        raise WebAuthnError("authenticator data is shorter than 37 bytes")
    out = {"rp_id_hash": data[:32], "flags": data[32], "sign_count": int.from_bytes(data[33:37], "big"),
           "user_present": bool(data[32] & 0x01), "user_verified": bool(data[32] & 0x04)}
    if data[32] & 0x40:                                  # AT: attested credential data follows
        if len(data) < 55:
            raise WebAuthnError("attested credential data is truncated")
        n = int.from_bytes(data[53:55], "big")
        if len(data) < 55 + n:
            raise WebAuthnError("credential id is truncated")
        out["aaguid"] = data[37:53]
        out["credential_id"] = data[55:55 + n]
        key, _ = cbor_decode(data, 55 + n)
        if not isinstance(key, dict):
            raise WebAuthnError("credential public key is not a COSE map")
        out["cose_key"] = key
    return out


def cose_es256_point(key: dict) -> bytes:
    """x || y (64 bytes) of a COSE EC2 P-256 key (kty 2, alg -7, crv 1)."""
    if key.get(1) != 2 or key.get(3) != ES256 or key.get(-1) != 1:
        raise WebAuthnError("only ES256 (P-256) credentials are supported")
    x, y = key.get(-2), key.get(-3)
    if not (isinstance(x, bytes) and isinstance(y, bytes) and len(x) == 32 and len(y) == 32):
        raise WebAuthnError("malformed EC2 coordinates")
    return x + y


def _verify_es256(point: bytes, signature_der: bytes, message: bytes) -> None:
    from cryptography.exceptions import InvalidSignature
    from cryptography.hazmat.primitives import hashes
    from cryptography.hazmat.primitives.asymmetric import ec
    try:
        pub = ec.EllipticCurvePublicNumbers(int.from_bytes(point[:32], "big"), int.from_bytes(point[32:], "big"),
                                            ec.SECP256R1()).public_key()
        pub.verify(signature_der, message, ec.ECDSA(hashes.SHA256()))
    except (InvalidSignature, ValueError) as e:
        raise WebAuthnError("signature does not verify") from e


class WebAuthnAuth:
    """Relying-party side of the two ceremonies.  Challenges are single-use and expire."""

    TIMEOUT_MS = 60000

    def __init__(self, rp_id: str = "localhost", rp_name: str = "AxonML", rp_origin: str = "http://localhost:3021"):
        self.rp_id, self.rp_name, self.rp_origin = rp_id, rp_name, rp_origin
        self._pending: dict[tuple[str, str], tuple[str, float]] = {}     # (kind, user id) -> (challenge, deadline)

    # ------------------------------------------------------------------ challenges
    def _issue(self, kind: str, user_id: str) -> str:
        challenge = b64u(os.urandom(32))
        self._pending[(kind, user_id)] = (challenge, time.time() + self.TIMEOUT_MS / 1000.0)
        return challenge

    def _take(self, kind: str, user_id: str) -> str:
        challenge, deadline = self._pending.pop((kind, user_id), (None, 0.0))
        if challenge is None or time.time() > deadline:
            raise WebAuthnError("no pending challenge (start the ceremony again)")
        return challenge

    def _client_data(self, raw: bytes, expect_type: str, challenge: str) -> None:
        try:
            cd = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WebAuthnError("clientDataJSON is not JSON") from e
        if cd.get("type") != expect_type:
            raise WebAuthnError(f"client data type is {cd.get('type')!r}, expected {expect_type!r}")
        if b64u_dec(str(cd.get("challenge", ""))) != b64u_dec(challenge):
            raise WebAuthnError("challenge mismatch")
        if str(cd.get("origin", "")).rstrip("/") != self.rp_origin.rstrip("/"):
            raise WebAuthnError(f"origin {cd.get('origin')!r} is not this relying party")

    def _rp_hash_ok(self, ad: dict) -> None:
        if ad["rp_id_hash"] != hashlib.sha256(self.rp_id.encode()).digest():
            raise WebAuthnError("relying-party id hash mismatch")
        if not ad["user_present"]:
            raise WebAuthnError("user-present flag is not set")

    # ------------------------------------------------------------------ registration
    def start_registration(self, user_id: str, user_name: str, display_name: str, exclude: list | None = None) -> dict:
        return {"challenge": self._issue("create", user_id),
                "rp": {"id": self.rp_id, "name": self.rp_name},
                "user": {"id": b64u(user_id.encode()), "name": user_name, "display_name": display_name},
                "pub_key_cred_params": [{"type": "public-key", "alg": ES256}],
                "timeout": self.TIMEOUT_MS, "attestation": "none",
                "exclude_credentials": [{"id": c["credential_id"], "type": "public-key"} for c in (exclude or [])],
                "authenticator_selection": {"authenticator_attachment": "cross-platform", "resident_key": "discouraged",
                                            "user_verification": "preferred"}}

    def finish_registration(self, user_id: str, response: dict, name: str) -> dict:
        challenge = self._take("create", user_id)
        resp = response.get("response") or {}
        try:
            cdj = b64u_dec(resp["client_data_json"])
            att, _ = cbor_decode(b64u_dec(resp["attestation_object"]))
        except KeyError as e:
            raise WebAuthnError(f"missing field {e.args[0]}") from e
        self._client_data(cdj, "webauthn.create", challenge)
        if not isinstance(att, dict) or not isinstance(att.get("authData"), bytes):
            raise WebAuthnError("attestation object has no authData")
        ad = parse_authenticator_data(att["authData"])
        self._rp_hash_ok(ad)
        if "cose_key" not in ad:
            raise WebAuthnError("no attested credential data")
        point = cose_es256_point(ad["cose_key"])
        fmt = att.get("fmt")
        if fmt == "packed":
            stmt = att.get("attStmt") or {}
            if "x5c" in stmt:
                raise WebAuthnError("attestation certificates are not evaluated; register with attestation 'none'")
            if stmt.get("alg") != ES256 or not isinstance(stmt.get("sig"), bytes):
                raise WebAuthnError("malformed packed self-attestation")
            _verify_es256(point, stmt["sig"], att["authData"] + hashlib.sha256(cdj).digest())
        elif fmt != "none":
            raise WebAuthnError(f"attestation format {fmt!r} is not accepted")
        cred_id = b64u(ad["credential_id"])
        if response.get("id") and b64u_dec(str(response["id"])) != ad["credential_id"]:
            raise WebAuthnError("credential id does not match the attested one")
        return {"credential_id": cred_id, "public_key": b64u(point), "counter": ad["sign_count"],
                "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "name": name or "security key"}

    # ------------------------------------------------------------------ authentication
    def start_authentication(self, user_id: str, credentials: list) -> dict:
        if not credentials:
            raise WebAuthnError("no registered credential")
        return {"challenge": self._issue("get", user_id), "timeout": self.TIMEOUT_MS, "rp_id": self.rp_id,
                "allow_credentials": [{"id": c["credential_id"], "type": "public-key"} for c in credentials],
                "user_verification": "preferred"}

    def finish_authentication(self, user_id: str, response: dict, credentials: list) -> dict:
        """Returns the matched credential with its counter advanced."""
        challenge = self._take("get", user_id)
        resp = response.get("response") or {}
        try:
            raw_id = b64u_dec(str(response.get("raw_id") or response["id"]))
            cdj = b64u_dec(resp["client_data_json"])
            adata = b64u_dec(resp["authenticator_data"])
            sig = b64u_dec(resp["signature"])
        except KeyError as e:
            raise WebAuthnError(f"missing field {e.args[0]}") from e
        cred = next((c for c in credentials if b64u_dec(c["credential_id"]) == raw_id), None)
        if cred is None:
            raise WebAuthnError("unknown credential")
        self._client_data(cdj, "webauthn.get", challenge)
        ad = parse_authenticator_data(adata)
        self._rp_hash_ok(ad)
        _verify_es256(b64u_dec(cred["public_key"]), sig, adata + hashlib.sha256(cdj).digest())
        old = int(cred.get("counter", 0))
        if (ad["sign_count"] or old) and ad["sign_count"] <= old:
            raise WebAuthnError("signature counter did not advance (cloned authenticator?)")
        return {**cred, "counter": ad["sign_count"]}


class SoftwareAuthenticator:
    """A P-256 software authenticator speaking the same wire shapes: the counterpart the tests and
    the command-line client use in place of a browser (``navigator.credentials``)."""

    def __init__(self, origin: str):
        self.origin = origin
        self._keys: dict[bytes, object] = {}
        self._counter = 0

    @staticmethod
    def _cose(pub) -> dict:
        n = pub.public_numbers()
        return {1: 2, 3: ES256, -1: 1, -2: n.x.to_bytes(32, "big"), -3: n.y.to_bytes(32, "big")}

    def _client_data(self, typ: str, challenge: str) -> bytes:
        return json.dumps({"type": typ, "challenge": challenge, "origin": self.origin, "crossOrigin": False}).encode()

    def create(self, options: dict) -> dict:
        from cryptography.hazmat.primitives.asymmetric import ec
        key = ec.generate_private_key(ec.SECP256R1())
        cred_id = os.urandom(32)
        self._keys[cred_id] = key
        rp_hash = hashlib.sha256(options["rp"]["id"].encode()).digest()
        auth_data = (rp_hash + bytes([0x41]) + (0).to_bytes(4, "big") + bytes(16) + len(cred_id).to_bytes(2, "big")
                     + cred_id + cbor_encode(self._cose(key.public_key())))
        cdj = self._client_data("webauthn.create", options["challenge"])
        att = cbor_encode({"fmt": "none", "attStmt": {}, "authData": auth_data})
        return {"id": b64u(cred_id), "raw_id": b64u(cred_id), "type": "public-key",
                "response": {"client_data_json": b64u(cdj), "attestation_object": b64u(att)}}

    def get(self, options: dict) -> dict:
        from cryptography.hazmat.primitives import hashes
        from cryptography.hazmat.primitives.asymmetric import ec
        cred_id = next((b64u_dec(c["id"]) for c in options["allow_credentials"] if b64u_dec(c["id"]) in self._keys), None)
        if cred_id is None:
            raise WebAuthnError("this authenticator holds none of the allowed credentials")
        self._counter += 1
        auth_data = hashlib.sha256(options["rp_id"].encode()).digest() + bytes([0x01]) + self._counter.to_bytes(4, "big")
        cdj = self._client_data("webauthn.get", options["challenge"])
        sig = self._keys[cred_id].sign(auth_data + hashlib.sha256(cdj).digest(), ec.ECDSA(hashes.SHA256()))
        return {"id": b64u(cred_id), "raw_id": b64u(cred_id), "type": "public-key",
                "response": {"client_data_json": b64u(cdj), "authenticator_data": b64u(auth_data),
                             "signature": b64u(sig), "user_handle": None}}
