"""Authentication for the platform server: password hashes, JWT access/refresh/MFA tokens, TOTP
second factor and single-use recovery codes, on the standard library only.

Parity: JWT claims ``sub/email/role/exp/iat/token_type/mfa_verified`` and the token pair / MFA
token shapes (crates/axonml-server/src/auth/jwt.rs:12-46, 84-227); TOTP SHA-1, 6 digits, 30 s
period, one step of tolerance (auth/totp.rs:84-98); ten ``NNNNN-NNNNN`` recovery codes stored only
as salted hashes and consumed on use (auth/recovery.rs:28-87); roles admin/user/viewer
(db/users.rs:16-27).  The WebAuthn second factor lives in ``webauthn.py``."""
from __future__ import annotations

import base64
import hashlib
import hmac
import json
import os
import secrets
import struct
import time
from dataclasses import dataclass


class AuthError(Exception):
    def __init__(self, message: str, status: int = 401):
        super().__init__(message)
        self.status = status


# ------------------------------------------------------------------ passwords
_PBKDF2_ITERS = 120_000


def hash_password(password: str, salt: bytes | None = None, iters: int = _PBKDF2_ITERS) -> str:
    salt = salt or os.urandom(16)
    dk = hashlib.pbkdf2_hmac("sha256", password.encode(), salt, iters)
    return f"pbkdf2_sha256${iters}${base64.b64encode(salt).decode()}${base64.b64encode(dk).decode()}"


def verify_password(password: str, stored: str) -> bool:
    try:
        scheme, iters, salt, dk = stored.split("$")
        if scheme != "pbkdf2_sha256":
            return False
        got = hashlib.pbkdf2_hmac("sha256", password.encode(), base64.b64decode(salt), int(iters))
        return hmac.compare_digest(got, base64.b64decode(dk))
    except (ValueError, TypeError):
        return False


# ------------------------------------------------------------------ JWT (HS256)
def _b64u(data: bytes) -> str:
    return base64.urlsafe_b64encode(data).rstrip(b"=").decode()


def _b64u_dec(s: str) -> bytes:
    return base64.urlsafe_b64decode(s + "=" * (-len(s) % 4))


@dataclass
class Claims:
    sub: str
    email: str
    role: str
    exp: int
    iat: int
    token_type: str = "access"
    mfa_verified: bool = False


class JwtAuth:
    def __init__(self, secret: str, access_expiry_hours: float = 24, refresh_expiry_days: float = 7):
        if len(secret) < 16:
            raise ValueError("JWT secret must have at least 16 characters")
        self._key = secret.encode()
        self.access_expiry_s = int(access_expiry_hours * 3600)
        self.refresh_expiry_s = int(refresh_expiry_days * 86400)

    def _encode(self, payload: dict) -> str:
        head = _b64u(json.dumps({"alg": "HS256", "typ": "JWT"}, separators=(",", ":")).encode())
        body = _b64u(json.dumps(payload, separators=(",", ":")).encode())
        sig = hmac.new(self._key, f"{head}.{body}".encode(), hashlib.sha256).digest()
        return f"{head}.{body}.{_b64u(sig)}"

    def _token(self, user_id, email, role, ttl, token_type, mfa_verified=False) -> str:
        now = int(time.time())
        # jti: two tokens issued to one user within the same second must differ, or revoking one
        # session (logout) would revoke the other too
        return self._encode({"sub": user_id, "email": email, "role": role, "exp": now + ttl, "iat": now,
                             "token_type": token_type, "mfa_verified": mfa_verified, "jti": secrets.token_hex(8)})

    def create_access_token(self, user_id, email, role, mfa_verified=False) -> str:
        return self._token(user_id, email, role, self.access_expiry_s, "access", mfa_verified)

    def create_refresh_token(self, user_id, email, role) -> str:
        return self._token(user_id, email, role, self.refresh_expiry_s, "refresh")

    def create_token_pair(self, user_id, email, role, mfa_verified=False) -> dict:
        return {"access_token": self.create_access_token(user_id, email, role, mfa_verified),
                "refresh_token": self.create_refresh_token(user_id, email, role),
                "expires_in": self.access_expiry_s, "token_type": "Bearer"}

    def create_mfa_token(self, user_id, email) -> dict:
        """Five-minute token that only the second-factor endpoints accept."""
        return {"mfa_token": self._token(user_id, email, "", 300, "mfa"), "expires_in": 300}

    def validate_token(self, token: str, token_type: str | None = None) -> Claims:
        try:
            head, body, sig = token.split(".")
            want = hmac.new(self._key, f"{head}.{body}".encode(), hashlib.sha256).digest()
            if not hmac.compare_digest(want, _b64u_dec(sig)):
                raise AuthError("invalid token signature")
            if json.loads(_b64u_dec(head)).get("alg") != "HS256":
                raise AuthError("unsupported token algorithm")
            p = json.loads(_b64u_dec(body))
            c = Claims(p["sub"], p.get("email", ""), p.get("role", ""), int(p["exp"]), int(p.get("iat", 0)),
                       p.get("token_type", ""), bool(p.get("mfa_verified", False)))
        except AuthError:
            raise
        except Exception as e:  # malformed token
            raise AuthError(f"malformed token: {type(e).__name__}") from None
        if c.exp < time.time():
            raise AuthError("token expired")
        if token_type is not None and c.token_type != token_type:
            raise AuthError(f"expected a {token_type} token")
        return c

    def validate_access_token(self, token):
        return self.validate_token(token, "access")

    def validate_refresh_token(self, token):
        return self.validate_token(token, "refresh")

    def validate_mfa_token(self, token):
        return self.validate_token(token, "mfa")

    def refresh_access_token(self, refresh_token: str) -> dict:
        c = self.validate_refresh_token(refresh_token)
        return self.create_token_pair(c.sub, c.email, c.role)

    @staticmethod
    def extract_from_header(header: str | None) -> str | None:
        if header and header.startswith("Bearer "):
            return header[7:].strip()
        return None


# ------------------------------------------------------------------ TOTP (RFC 6238)
class TotpAuth:
    def __init__(self, issuer: str = "AxonML", digits: int = 6, period: int = 30, skew: int = 1):
        self.issuer, self.digits, self.period, self.skew = issuer, digits, period, skew

    @staticmethod
    def generate_secret() -> str:
        return base64.b32encode(os.urandom(20)).decode().rstrip("=")

    def _code(self, secret: str, counter: int) -> str:
        key = base64.b32decode(secret + "=" * (-len(secret) % 8), casefold=True)
        mac = hmac.new(key, struct.pack(">Q", counter), hashlib.sha1).digest()
        off = mac[-1] & 0xF
        val = struct.unpack(">I", mac[off:off + 4])[0] & 0x7FFFFFFF
        return str(val % 10 ** self.digits).zfill(self.digits)

    def code_at(self, secret: str, t: float | None = None) -> str:
        return self._code(secret, int((time.time() if t is None else t) // self.period))

    def verify(self, secret: str, code: str, t: float | None = None) -> bool:
        code = code.strip().replace(" ", "")
        c = int((time.time() if t is None else t) // self.period)
        return any(hmac.compare_digest(self._code(secret, c + d), code) for d in range(-self.skew, self.skew + 1))

    def setup(self, user_email: str) -> dict:
        from urllib.parse import quote
        secret = self.generate_secret()
        uri = (f"otpauth://totp/{quote(self.issuer)}:{quote(user_email)}?secret={secret}&issuer={quote(self.issuer)}"
               f"&algorithm=SHA1&digits={self.digits}&period={self.period}")
        return {"secret": secret, "otpauth_url": uri}


# ------------------------------------------------------------------ recovery codes
class RecoveryAuth:
    @staticmethod
    def _hash(code: str, salt: bytes | None = None) -> str:
        return hash_password(code.replace("-", ""), salt, iters=20_000)

    @classmethod
    def generate_codes(cls, count: int = 10) -> dict:
        codes = [f"{secrets.randbelow(100000):05d}-{secrets.randbelow(100000):05d}" for _ in range(count)]
        return {"codes": codes, "hashed_codes": [cls._hash(c) for c in codes]}

    @staticmethod
    def verify_code(code: str, stored_hashes: list[str]) -> int | None:
        """Index of the matching stored hash (the caller removes it: a code works once)."""
        plain = code.strip().replace("-", "")
        for i, h in enumerate(stored_hashes):
            if verify_password(plain, h):
                return i
        return None

    @staticmethod
    def format_for_display(codes: list[str]) -> str:
        return "\n".join(f"{i + 1:2d}. {c}" for i, c in enumerate(codes))


ROLES = ("admin", "user", "viewer")


def require_role(claims: Claims, *allowed: str) -> None:
    if claims.role not in allowed:
        raise AuthError(f"role {claims.role!r} may not do this", status=403)
