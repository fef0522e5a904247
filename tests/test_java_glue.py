"""The Java glue without a JDK: what `javac -h` and a C compiler would check.

No JDK or JNI headers exist in this build image, so the Java layer cannot be compiled here.  These tests hold the
three files that must agree against one another instead:

* every ``native`` method of ``OmoeNative.java`` has exactly one ``JFN(...)`` definition in ``omoe_jni.c`` with the
  JNI name, return type and parameter types ``javac -h`` would generate for it (naming as in the reference's own
  JNI header, jni/com_omega_engine_gpu_JNITest.h:15-32), and the shim defines nothing else;
* ``omoe_jni.c`` compiles (``-fsyntax-only -Wall -Werror``) against ``include/omoe.h`` and a minimal stand-in for
  ``jni.h`` that the test writes (types, macros and the handful of JNIEnv functions the shim uses), so every C-ABI
  call in it has the right arity and pointer types;
* every ``OmoeNative.x(...)`` call in ``MoELayer.java`` names a declared native and passes as many arguments as it
  takes, and the layer overrides the operator surface the transformer block drives
  (src/main/java/com/omega/engine/nn/layer/Layer.java:66-104; LlamaTransformerBlock.java:277-289).
"""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JAVA = os.path.join(ROOT, "omega_ai_b200", "java")
NATIVE = os.path.join(JAVA, "com", "omega", "engine", "nn", "layer", "llama", "OmoeNative.java")
LAYER = os.path.join(JAVA, "com", "omega", "engine", "nn", "layer", "llama", "MoELayer.java")
SHIM = os.path.join(JAVA, "jni", "omoe_jni.c")

JNI_TYPE = {"int": "jint", "long": "jlong", "float": "jfloat", "String": "jstring", "float[]": "jfloatArray",
            "int[]": "jintArray", "long[]": "jlongArray", "byte[]": "jbyteArray", "void": "void"}

JNI_H = r"""
#ifndef FAKE_JNI_H
#define FAKE_JNI_H
#include <stdint.h>
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_ABORT 2
typedef int32_t jint; typedef int64_t jlong; typedef float jfloat; typedef int8_t jbyte; typedef jint jsize;
typedef struct _jobject *jobject; typedef jobject jclass; typedef jobject jstring; typedef jobject jarray;
typedef jarray jfloatArray; typedef jarray jintArray; typedef jarray jlongArray; typedef jarray jbyteArray;
typedef unsigned char jboolean;
struct JNINativeInterface_;
typedef const struct JNINativeInterface_ *JNIEnv;
struct JNINativeInterface_ {
    jstring (*NewStringUTF)(JNIEnv *, const char *);
    jsize (*GetArrayLength)(JNIEnv *, jarray);
    jobject (*NewGlobalRef)(JNIEnv *, jobject);
    void (*DeleteGlobalRef)(JNIEnv *, jobject);
    jfloat *(*GetFloatArrayElements)(JNIEnv *, jfloatArray, jboolean *);
    void (*ReleaseFloatArrayElements)(JNIEnv *, jfloatArray, jfloat *, jint);
    jint *(*GetIntArrayElements)(JNIEnv *, jintArray, jboolean *);
    void (*ReleaseIntArrayElements)(JNIEnv *, jintArray, jint *, jint);
    jlong *(*GetLongArrayElements)(JNIEnv *, jlongArray, jboolean *);
    void (*ReleaseLongArrayElements)(JNIEnv *, jlongArray, jlong *, jint);
    jbyte *(*GetByteArrayElements)(JNIEnv *, jbyteArray, jboolean *);
    void (*ReleaseByteArrayElements)(JNIEnv *, jbyteArray, jbyte *, jint);
};
#endif
"""


def _strip_comments(src):
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    return re.sub(r"//[^\n]*", " ", src)


def java_natives():
    src = _strip_comments(open(NATIVE).read())
    out = {}
    for m in re.finditer(r"public\s+static\s+native\s+([\w\[\]]+)\s+(\w+)\s*\(([^)]*)\)\s*;", src):
        ret, name, params = m.group(1), m.group(2), m.group(3)
        types = []
        for prm in [p.strip() for p in params.split(",") if p.strip()]:
            t = prm.rsplit(None, 1)[0].replace(" ", "")
            types.append(t)
        assert name not in out, f"overloaded native {name}: JNI names would need mangled signatures"
        out[name] = (ret, types)
    return out


def shim_functions():
    src = _strip_comments(open(SHIM).read())
    out = {}
    for m in re.finditer(r"JFN\(\s*(\w+)\s*,\s*(\w+)\s*\)\s*\(([^)]*)\)", src):
        ret, name, params = m.group(1), m.group(2), m.group(3)
        ps = [p.strip() for p in params.split(",")]
        assert ps[0].replace(" ", "") == "JNIEnv*env" and ps[1].split()[0] == "jclass", f"{name}: static natives take (JNIEnv*, jclass, ...)"
        types = [p.rsplit(None, 1)[0].strip() for p in ps[2:]]
        assert name not in out
        out[name] = (ret, types)
    return out


def test_every_native_has_its_jni_definition():
    natives, shim = java_natives(), shim_functions()
    assert len(natives) >= 15
    assert set(natives) == set(shim), (sorted(set(natives) - set(shim)), sorted(set(shim) - set(natives)))
    for name, (ret, types) in natives.items():
        want = (JNI_TYPE[ret], [JNI_TYPE[t] for t in types])
        assert shim[name] == want, f"{name}: Java declares {want}, the shim defines {shim[name]}"
    macro = re.search(r"#define\s+JFN\(ret,\s*name\)\s+JNIEXPORT ret JNICALL (\w+)##name", open(SHIM).read())
    assert macro and macro.group(1) == "Java_com_omega_engine_nn_layer_llama_OmoeNative_"
    pkg = re.search(r"package\s+([\w.]+);", open(NATIVE).read()).group(1)
    assert "Java_" + pkg.replace(".", "_") + "_OmoeNative_" == macro.group(1)


def test_shim_compiles_against_the_c_abi(tmp_path):
    (tmp_path / "jni.h").write_text(JNI_H)
    cmd = ["gcc", "-std=c11", "-fsyntax-only", "-Wall", "-Werror", "-I", str(tmp_path),
           "-I", os.path.join(ROOT, "include"), SHIM]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    # and the guard really took the JNI branch (a shim that compiled to nothing would pass the line above)
    p = subprocess.run(["gcc", "-std=c11", "-E", "-dM", "-I", str(tmp_path), "-I", os.path.join(ROOT, "include"), SHIM],
                       capture_output=True, text=True)
    assert "OMOE_HAVE_JNI" in p.stdout


def _call_arity(src, start):
    depth, n, i, seen = 0, 0, start, False
    while True:
        ch = src[i]
        if ch == "(":
            depth += 1
        elif ch == ")":
            depth -= 1
            if depth == 0:
                return n + (1 if seen else 0)
        elif ch == "," and depth == 1:
            n += 1
        elif depth >= 1 and not ch.isspace():
            seen = True
        i += 1


def test_layer_calls_match_the_natives_and_cover_the_operator_surface():
    natives = java_natives()
    src = _strip_comments(open(LAYER).read())
    calls = list(re.finditer(r"OmoeNative\.(\w+)\s*\(", src))
    assert calls
    for m in calls:
        name = m.group(1)
        assert name in natives, f"MoELayer.java calls OmoeNative.{name}, which is not declared"
        got = _call_arity(src, m.end() - 1)
        assert got == len(natives[name][1]), f"OmoeNative.{name}: {got} arguments passed, {len(natives[name][1])} declared"
    assert re.search(r"class\s+MoELayer\s+extends\s+Layer", src)
    for method in ("init", "initParam", "output", "forward", "getOutput", "diff", "back", "update", "accGrad",
                   "saveModel", "loadModel", "putParamters", "putParamterGrads", "getLayerType", "initBack"):
        assert re.search(r"public\s+[\w\[\]]+\s+" + method + r"\s*\(", src), f"MoELayer.java lacks {method}()"
    assert "LayerType.feed_forward" in src
